"""Benchmark of the sm_100a attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--samples R] [--impl ours|reference] [--workload decode_q1]

One "step" is one call of ``atrex.flash_attn_varlen_func`` over one synthetic batch.
The default workload is the BF16 Q1 paged decode configuration (batch 64, 32 query /
8 KV heads, head_dim 128, page 64, KV lengths uniform in [1024, 16384], block table =
seeded permutation of a 20000-page pool, N(0,1) inputs, num_splits = 0).  Its metric
is achieved HBM GB/s on ALGORITHMIC bytes: the K and V rows every query can see, plus
Q, O and the page-table entries read.  Prefill workloads report TFLOP/s on algorithmic
FLOPs (4 * D * Hq * visible pairs).

The JSON line's top-level keys describe the chosen workload; with the default workload
the same process then measures the other configurations of the metric (speculative
decode, FP8 head_dim-256 prefill, BF16 head_dim-128 prefill, the request-sharded
256-request prefill set) and reports them under ``sub_results`` with their own
roofline, end-to-end and clock records.

Protocol (the reference's harness takes the median of 31 samples of 20 calls,
op_test/nvidia/flash_attn/test_flash_attn_sm103.py:1061-1087): W warm-up steps, then R
samples (default 7) of exactly K steps each, every sample bracketed by a barrier and a
device synchronise and timed with CUDA events; per sample the MAXIMUM over ranks counts;
``ms_per_step`` / ``value`` come from the median sample and ``spread`` gives min and max.

With N > 1 the requests of all ranks (N batches for a "weak" workload, one fixed set for
the "strong" one) are pooled and dealt to the ranks by cost, longest first
(``sharding.partition_requests``); every rank derives the same partition.  No collective
is on the data path of the request-sharded workloads; ``decode_q1_headsplit`` (KV heads
split over the ranks, O all-gathered) and ``decode_cp`` (every request's keys dealt to
the ranks, (O, LSE) gathered and merged) are the variants with a real exchange step.

``--impl reference`` times the CPU FP32 attention (the oracle port of the reference's
``reference()`` in op_test/utils/flash_attn_contract.py:81-111) on the host cores on a
bounded sample of the same workload and prints the same JSON shape.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
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
    "decode_q1": dict(kind="decode", batch=64, q_len=1, hq=32, hkv=8, d=128, page=64, kv_lo=1024, kv_hi=16384,
                      pool=20000, window=None, sink=False, lse=False, scaling="weak"),
    # same shape at a quarter of the batch and a small pool: the case profiler captures run on
    "decode_q1_small": dict(kind="decode", batch=16, q_len=1, hq=32, hkv=8, d=128, page=64, kv_lo=1024,
                            kv_hi=16384, pool=2500, window=None, sink=False, lse=False, scaling="weak"),
    # BF16 speculative decode, query length 4, sliding window, sinks, LSE
    "decode_q4_window": dict(kind="decode", batch=128, q_len=4, hq=64, hkv=4, d=128, page=128, kv_lo=32768,
                             kv_hi=32768, pool=128 * 256 + 64, window=(4095, 0), sink=True, lse=True,
                             scaling="weak"),
    # BF16 causal paged prefill, head_dim 128, query = full KV; lengths log-normal (median 8192, sigma 0.75,
    # clipped to [1024, 131072]).  "prefill_hd128" is a 16-request batch per GPU; "prefill_sharded" is one fixed
    # 256-request set sharded over the ranks by request, FLOP-balanced.
    "prefill_hd128": dict(kind="prefill", batch=16, hq=64, hkv=8, d=128, page=64, median=8192, sigma=0.75,
                          clip=(1024, 131072), window=None, sink=False, lse=False, scaling="weak"),
    "prefill_small": dict(kind="prefill", batch=4, hq=64, hkv=8, d=128, page=64, median=4096, sigma=0.5,
                          clip=(1024, 16384), window=None, sink=False, lse=False, scaling="weak"),
    # two requests of 32768 tokens: the long-request case profiler captures run on (K/V of one KV head = 16 MB)
    "prefill_long2": dict(kind="prefill", batch=2, hq=64, hkv=8, d=128, page=64, median=32768, sigma=0.0,
                          clip=(32768, 32768), window=None, sink=False, lse=False, scaling="weak"),
    # FP8 E4M3 causal paged prefill with a cached prefix, head_dim 256, per-(request, KV head) descales = amax / 448
    "prefill_fp8_hd256": dict(kind="prefill", batch=16, hq=24, hkv=2, d=256, page=128, q_range=(512, 4096),
                              prefix_range=(0, 4096), fp8=True, window=None, sink=False, lse=False, scaling="weak"),
    # small cases of the same kernels for profiler captures
    "prefill_fp8_small": dict(kind="prefill", batch=4, hq=24, hkv=2, d=256, page=128, q_range=(512, 2048),
                              prefix_range=(0, 2048), fp8=True, window=None, sink=False, lse=False, scaling="weak"),
    "decode_q4_small": dict(kind="decode", batch=32, q_len=4, hq=64, hkv=4, d=128, page=128, kv_lo=32768,
                            kv_hi=32768, pool=32 * 256 + 64, window=(4095, 0), sink=True, lse=True,
                            scaling="weak"),
    # KV-cache write path (the step before attention): one prefill chunk of new tokens scattered into the paged
    # pools, BF16 cache and FP8 E4M3 cache (per-head scales); 0.5 GB of K/V rows per step (4x L2)
    "kv_write": dict(kind="kv_write", tokens=131072, hkv=8, d=128, page=64, fp8=False, scaling="weak"),
    "kv_write_fp8": dict(kind="kv_write", tokens=131072, hkv=8, d=128, page=64, fp8=True, scaling="weak"),
    # the same with the per-head scales computed from the step's rows first (max |x| / 448): two passes over K/V
    "kv_write_fp8_scaled": dict(kind="kv_write", tokens=131072, hkv=8, d=128, page=64, fp8=True, scales="computed",
                                scaling="weak"),
    "kv_write_small": dict(kind="kv_write", tokens=65536, hkv=8, d=128, page=64, fp8=False, scaling="weak"),
    # variants with an exchange step (N >= 2): the decode batch with the KV heads split over the ranks and O
    # all-gathered; 16 requests of 131072 keys whose keys are dealt to the ranks (context parallelism)
    "decode_q1_headsplit": dict(kind="decode", batch=64, q_len=1, hq=32, hkv=8, d=128, page=64, kv_lo=1024,
                                kv_hi=16384, pool=20000, window=None, sink=False, lse=False, scaling="strong",
                                variant="headsplit"),
    "decode_cp": dict(kind="decode", batch=16, q_len=1, hq=32, hkv=8, d=128, page=64, kv_lo=131072, kv_hi=131072,
                      pool=None, window=None, sink=False, lse=True, scaling="strong", variant="cp"),
    # compact sparse attention (atrex.qsa_compact): query-length-1 decode rows that each list 512 four-token blocks
    # of their own request's 65536-token cache (head_dim 256, 8 query heads on 1 KV head, page 128): a gather of
    # 2 KB pieces, 2.1 MB per row in BF16; and a ragged prefill chunk of one request
    "qsa_decode": dict(kind="qsa", rows=64, requests=64, tokens=65536, hq=8, hkv=1, page=128, fp8=False, scaling="weak"),
    "qsa_decode_fp8": dict(kind="qsa", rows=64, requests=64, tokens=65536, hq=8, hkv=1, page=128, fp8=True,
                           scaling="weak"),
    "qsa_decode_small": dict(kind="qsa", rows=16, requests=16, tokens=65536, hq=8, hkv=1, page=128, fp8=False,
                             scaling="weak"),   # the case profiler captures run on (1.1 GB of cache)
    "qsa_prefill": dict(kind="qsa", rows=2048, requests=1, tokens=32768, hq=8, hkv=1, page=128, fp8=False,
                        scaling="weak"),
    "qsa_prefill_fp8": dict(kind="qsa", rows=2048, requests=1, tokens=32768, hq=8, hkv=1, page=128, fp8=True,
                            scaling="weak"),
    "prefill_sharded": dict(kind="prefill", batch=256, hq=64, hkv=8, d=128, page=64, median=8192, sigma=0.75,
                            clip=(1024, 131072), window=None, sink=False, lse=False, scaling="strong"),
}
# DRAM bytes per algorithmic byte of the dominant kernel, from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum on the small case of the same kernel; traffic grows in proportion
# to the K/V bytes a launch reads, so the ratio carries to the full-size launch).
NCU_TRAFFIC_RATIO = {"kv_write": 1.0, "kv_write_small": 1.0, "kv_write_fp8": 1.0,
                     "decode_q1": 1.0250, "decode_q1_small": 1.0250, "decode_q4_window": 1.0553, "decode_q4_small": 1.0553,
                     "qsa_decode": 1.0226, "qsa_decode_fp8": 1.0114, "qsa_decode_small": 1.0}
# The tensor-bound BF16 prefill kernel: DRAM bytes per byte of (Q + O + K + V), from the captures of prefill_small
# (0.963) and of two 32768-token requests (0.988); K/V re-reads are served by L2.
NCU_PREFILL_IO_RATIO = {"prefill_small": 0.963, "prefill_long2": 0.988, "prefill_hd128": 0.988, "prefill_sharded": 0.988}
E2E_MAX_BYTES = 8 << 30   # largest Q the end-to-end leg stages in pinned host memory
KIND = {
    "decode": dict(metric="paged_decode_hbm_bandwidth", unit="GB/s", scale=1e9, bound="hbm"),
    "prefill": dict(metric="paged_prefill_tensor_throughput", unit="TFLOP/s", scale=1e12, bound="tensor"),
    "kv_write": dict(metric="kv_cache_write_hbm_bandwidth", unit="GB/s", scale=1e9, bound="hbm"),
    "qsa": dict(metric="sparse_attention_gather_bandwidth", unit="GB/s", scale=1e9, bound="hbm"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            data = json.load(f)
        return dict(hbm=float(data["hbm_gbs"]), tensor=float(data["bf16_tflops_sustained"]),
                    tensor_burst=float(data["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


def draw_lengths(spec, seed):
    """(q_lens, kv_lens) of one batch."""
    rng = np.random.default_rng(seed)
    if spec["kind"] == "decode":
        kv = rng.integers(spec["kv_lo"], spec["kv_hi"] + 1, size=spec["batch"]).tolist()
        return [spec["q_len"]] * spec["batch"], kv
    if "q_range" in spec:
        q = rng.integers(spec["q_range"][0], spec["q_range"][1] + 1, size=spec["batch"])
        prefix = rng.integers(spec["prefix_range"][0], spec["prefix_range"][1] + 1, size=spec["batch"])
        return q.tolist(), (q + prefix).tolist()
    raw = np.exp(rng.normal(np.log(spec["median"]), spec["sigma"], spec["batch"]))
    kv = np.clip(np.round(raw), *spec["clip"]).astype(int).tolist()
    return list(kv), list(kv)


# ---- work accounting (the benchmark's own; tests/test_bench_accounting.py checks it against the oracle's) ----
def causal_visible_pairs(q_len, kv_len, left=-1):
    """(query, key) pairs a causal call does not mask: query i sees keys [max(0, i + off - left), i + off],
    off = kv_len - q_len (bottom-right aligned); left < 0 = no sliding window."""
    off = kv_len - q_len
    total = 0
    for i in range(q_len):
        hi = min(kv_len - 1, i + off)
        lo = 0 if left < 0 else max(0, i + off - left)
        total += max(0, hi - lo + 1)
    return total


def algorithmic_flops(q_lens, kv_lens, num_q_heads, head_dim, left=-1):
    """4 * D * Hq * visible pairs: 2 FLOP per multiply-add in Q K^T and in P V."""
    pairs = 0
    for nq, nk in zip(q_lens, kv_lens):
        if left < 0 and nk >= nq:
            pairs += nq * (nk - nq) + nq * (nq + 1) // 2          # closed form of the sum above
        else:
            pairs += causal_visible_pairs(nq, nk, left)
    return 4 * head_dim * num_q_heads * pairs


def algorithmic_decode_bytes(q_lens, kv_lens, num_q_heads, num_kv_heads, head_dim, elem_bytes, page_size, left=-1):
    """K + V bytes of the keys any query row of a request can see, its page-table entries, Q read and O written."""
    total = 0
    for nq, nk in zip(q_lens, kv_lens):
        span = nk if left < 0 else min(nk, left + nq)
        total += span * num_kv_heads * head_dim * 2 * elem_bytes
        total += 4 * math.ceil(span / page_size)
        total += nq * num_q_heads * head_dim * (elem_bytes + 2)
    return total


def kv_write_bytes(tokens, num_kv_heads, head_dim, fp8):
    """K and V rows read as BF16 and written once in the cache's element size, plus the 8-byte slot ids."""
    row = num_kv_heads * head_dim
    return tokens * (2 * row * 2 + 2 * row * (1 if fp8 else 2) + 8)


def work_units(spec, q_lens, kv_lens):
    """Algorithmic bytes (decode) or FLOPs (prefill) of one pass over the batch."""
    left = spec["window"][0] if spec["window"] else -1
    if spec["kind"] == "decode":
        total = algorithmic_decode_bytes(q_lens, kv_lens, spec["hq"], spec["hkv"], spec["d"], 2, spec["page"], left)
        if spec["lse"]:
            total += 4 * sum(q_lens) * spec["hq"]
        return total
    return algorithmic_flops(q_lens, kv_lens, spec["hq"], spec["d"], left)

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


def build_device_case(spec, q_lens, kv_lens, seed, device):
    """Synthetic batch resident on ``device`` plus pinned host copies of the per-step inputs."""
    import torch

    g = torch.Generator(device=device).manual_seed(seed)
    page, hkv, d = spec["page"], spec["hkv"], spec["d"]
    counts = [-(-n // page) for n in kv_lens]
    pool = spec.get("pool") or sum(counts) + 8
    k = torch.randn((pool, page, hkv, d), generator=g, device=device, dtype=torch.bfloat16)
    v = torch.randn((pool, page, hkv, d), generator=g, device=device, dtype=torch.bfloat16)
    total_q = sum(q_lens)
    q = torch.randn((total_q, spec["hq"], d), generator=g, device=device, dtype=torch.bfloat16)
    width = max(counts + [1])
    rng = np.random.default_rng(seed + 1)
    perm = rng.permutation(pool).astype(np.int32)
    table = np.full((len(counts), width), -1, dtype=np.int32)
    o = 0
    for r, n in enumerate(counts):
        table[r, :n] = perm[o:o + n]
        o += n
    assert o <= pool
    cu = np.zeros(len(q_lens) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(q_lens)
    # end-to-end legs copy Q from pinned host memory every step; beyond a few GB that leg is skipped (see main)
    big = q.numel() * q.element_size() > E2E_MAX_BYTES
    host = dict(
        q=q[:1].cpu().pin_memory() if big else q.cpu().pin_memory(),
        cu_seqlens_q=torch.from_numpy(cu).pin_memory(),
        seqused_k=torch.tensor(kv_lens, dtype=torch.int32).pin_memory(),
        block_table=torch.from_numpy(table).pin_memory(),
    )
    descales = {}
    if spec.get("fp8"):
        # quantise as a serving stack would: one scale per (request, KV head) from that request's own tokens
        group = spec["hq"] // hkv
        table_d = torch.from_numpy(table).to(device)
        kq, vq = torch.empty_like(k, dtype=torch.float8_e4m3fn), torch.empty_like(v, dtype=torch.float8_e4m3fn)
        qq = torch.empty_like(q, dtype=torch.float8_e4m3fn)
        for name in ("q_descale", "k_descale", "v_descale"):
            descales[name] = torch.empty((len(q_lens), hkv), dtype=torch.float32, device=device)
        for r, n in enumerate(counts):
            ids = table_d[r, :n].long()
            for src, dst, name in ((k, kq, "k_descale"), (v, vq, "v_descale")):
                block = src[ids].float()
                scale = block.abs().amax(dim=(0, 1, 3)).clamp_min(1e-6) / 448.0
                dst[ids] = (block / scale[None, None, :, None]).to(torch.float8_e4m3fn)
                descales[name][r] = scale
            rows = q[cu[r]:cu[r + 1]].float().view(q_lens[r], hkv, group, d)
            scale = rows.abs().amax(dim=(0, 2, 3)).clamp_min(1e-6) / 448.0
            qq[cu[r]:cu[r + 1]] = (rows / scale[None, :, None, None]).view(q_lens[r], spec["hq"], d).to(torch.float8_e4m3fn)
            descales["q_descale"][r] = scale
        k, v, q = kq, vq, qq
        host["q"] = (q[:1] if big else q).view(torch.uint8).cpu().pin_memory().view(torch.float8_e4m3fn)
    case = dict(q=q, k=k, v=v, max_seqlen_q=max(q_lens + [0]), cu_seqlens_q=host["cu_seqlens_q"].to(device),
                max_seqlen_k=width * page, seqused_k=host["seqused_k"].to(device),
                block_table=host["block_table"].to(device), softmax_scale=d ** -0.5, causal=True,
                window_size=spec["window"], num_splits=0, return_softmax_lse=spec["lse"],
                out=torch.empty(q.shape, dtype=torch.bfloat16, device=device), **descales)
    if spec["sink"]:
        case["s_aux"] = torch.randn(spec["hq"], generator=g, device=device).bfloat16()
    return case, host


def cpu_threads():
    try:
        from threadpoolctl import threadpool_info

        return max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        return os.cpu_count() or 1


def cpu_baseline(spec, q_lens, kv_lens, seed, budget_s=12.0):
    """The CPU FP32 oracle over requests of the workload (shortest first for prefill) until about ``budget_s``
    seconds are used.  Returns (cpu_baseline dict, seconds)."""
    from oracle import fa_oracle

    kind = KIND[spec["kind"]]
    rng = np.random.default_rng(seed)
    hq, hkv, d, page = spec["hq"], spec["hkv"], spec["d"], spec["page"]
    window = spec["window"] or (-1, -1)
    order = range(len(kv_lens)) if spec["kind"] == "decode" else np.argsort(kv_lens).tolist()
    done, n_req, t_total = 0, 0, 0.0
    for b in order:
        nq, n = q_lens[b], kv_lens[b]
        if spec["kind"] == "prefill" and n_req >= 1 and t_total > 0 and t_total * (1 + (n / kv_lens[order[0]]) ** 2) > 2.5 * budget_s:
            break
        pages = -(-n // page)
        k = fa_oracle.bf16_round(rng.standard_normal((pages, page, hkv, d), dtype=np.float32))
        v = fa_oracle.bf16_round(rng.standard_normal((pages, page, hkv, d), dtype=np.float32))
        q = fa_oracle.bf16_round(rng.standard_normal((nq, hq, d), dtype=np.float32))
        table = np.arange(pages, dtype=np.int32)[None, :]
        sink = rng.standard_normal(hq).astype(np.float32) if spec["sink"] else None
        t0 = time.perf_counter()
        fa_oracle.attention(q, k, v, np.array([0, nq], np.int32), seqused_k=np.array([n], np.int32),
                            block_table=table, softmax_scale=d ** -0.5, causal=True, window=window, sink=sink)
        t_total += time.perf_counter() - t0
        done += work_units(spec, [nq], [n])
        n_req += 1
        if t_total >= budget_s:
            break
    which = "first" if spec["kind"] == "decode" else "shortest"
    return dict(value=done / t_total / kind["scale"], unit=kind["unit"], cores=cpu_threads(), kind="port",
                sample=f"{which} {n_req} of {len(kv_lens)} requests of the workload, one pass, {t_total:.1f} s"), t_total


def run_reference(args, spec, rank, world):
    """CPU arm: each step is the oracle over a bounded sample of the batch."""
    if rank != 0:
        return
    kind = KIND[spec["kind"]]
    steps, warm = max(1, args.steps), max(0, args.warmup)
    per_step = max(2.0, min(20.0, 120.0 / (steps + warm)))
    if spec["kind"] == "qsa":
        raise SystemExit("the CPU arm of the sparse attention workloads is their cpu_baseline (run without --impl)")
    if spec["kind"] == "kv_write":
        values, sample, total_t = [], None, 0.0
        for _ in range(min(steps, 8)):
            sample, t = kv_write_cpu(spec, 1729, per_step)
            values.append(sample["value"])
            total_t += t
        value = statistics.median(values)
        print(json.dumps(dict(
            impl="reference", metric=kind["metric"], value=value, unit=kind["unit"], n_gpus=args.gpus,
            steps=len(values), warmup=0, ms_per_step=total_t / len(values) * 1e3, higher_is_better=True,
            scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
            config=dict(workload=args.workload, new_tokens=spec["tokens"], num_kv_heads=spec["hkv"],
                        head_dim=spec["d"], page_size=spec["page"]),
            cpu_baseline=dict(sample, value=value),
            e2e=dict(value=value, unit=kind["unit"], h2d_bytes_per_step=0, d2h_bytes_per_step=0))))
        return
    q_lens, kv_lens = draw_lengths(spec, 1729)
    for _ in range(min(warm, 1)):
        cpu_baseline(spec, q_lens, kv_lens, 1729, budget_s=1.0)
    values, sample, total_t = [], None, 0.0
    for _ in range(min(steps, 8)):
        sample, t = cpu_baseline(spec, q_lens, kv_lens, 1729, budget_s=per_step)
        values.append(sample["value"])
        total_t += t
    value = statistics.median(values)
    line = dict(impl="reference", metric=kind["metric"], value=value, unit=kind["unit"], n_gpus=args.gpus,
                steps=len(values), warmup=min(warm, 1), ms_per_step=total_t / len(values) * 1e3,
                higher_is_better=True, scaling=spec["scaling"], vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=args.workload, **{k: spec[k] for k in ("batch", "hq", "hkv", "d", "page")}),
                cpu_baseline=dict(sample, value=value),
                e2e=dict(value=value, unit=kind["unit"], h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def kv_write_inputs(spec, seed, device, torch):
    """One step's new K/V rows, empty pools and a slot mapping that fills random pages (a block table's order)."""
    tokens, hkv, d, page = spec["tokens"], spec["hkv"], spec["d"], spec["page"]
    pages = tokens // page + 64
    g = torch.Generator(device=device).manual_seed(seed)
    key = torch.randn(tokens, hkv, d, device=device, generator=g).bfloat16()
    value = torch.randn(tokens, hkv, d, device=device, generator=g).bfloat16()
    dtype = torch.float8_e4m3fn if spec["fp8"] else torch.bfloat16
    cache = torch.zeros(pages, 2, page, hkv, d, dtype=torch.uint8 if spec["fp8"] else dtype, device=device)
    if spec["fp8"]:
        cache = cache.view(dtype)
    page_order = torch.randperm(pages, device=device, generator=g)[: tokens // page]
    slots = (page_order[:, None] * page + torch.arange(page, device=device)[None, :]).reshape(-1).to(torch.int64)
    scales = None
    if spec["fp8"]:
        scales = (0.5 + 0.125 * torch.arange(hkv, dtype=torch.float32, device=device),
                  1.0 + 0.0625 * torch.arange(hkv, dtype=torch.float32, device=device))
    return key, value, cache[:, 0], cache[:, 1], slots, scales


def kv_write_cpu(spec, seed, budget_s):
    """The oracle's scatter (numpy, one thread) over a bounded sample of the step's tokens."""
    import numpy as np
    from oracle import kv_cache_oracle
    hkv, d, page = spec["hkv"], spec["d"], spec["page"]
    rng = np.random.default_rng(seed)
    sample = 4096
    key = rng.standard_normal((sample, hkv, d), dtype=np.float32)
    value = rng.standard_normal((sample, hkv, d), dtype=np.float32)
    slots = rng.permutation(sample).astype(np.int64)
    kc = np.zeros((sample // page, page, hkv, d), dtype=np.float32)
    vc = np.zeros_like(kc)
    scale = np.linspace(0.5, 1.5, hkv).astype(np.float32)
    done, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < budget_s:
        kv_cache_oracle.write_kv_cache(key, value, kc, vc, slots, scale, scale, fp8=spec["fp8"])
        done += sample
    t = time.perf_counter() - t0
    work = kv_write_bytes(done, hkv, d, spec["fp8"])
    return dict(value=work / t / 1e9, unit="GB/s", cores=1, kind="port",
                sample=f"oracle scatter of {done} of the step's {spec['tokens']} tokens, {t:.1f} s"), t


def run_kv_write(args, spec, rank, world, local):
    """KV-cache write workload: same JSON contract, the kernel timed by CUDA events around each call."""
    import torch
    import torch.distributed as dist
    from atrex.src.nvidia.flash_attn.sm100 import kv_cache, runtime

    kind = KIND["kv_write"]
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    runtime.prewarm(device)
    key, value, kc, vc, slots, scales = kv_write_inputs(spec, 1729 + 1000 * rank, device, torch)
    ks, vs = scales if scales else (None, None)
    work = kv_write_bytes(spec["tokens"], spec["hkv"], spec["d"], spec["fp8"])
    computed = spec.get("scales") == "computed"
    if computed:
        work += spec["tokens"] * spec["hkv"] * spec["d"] * 2 * 2      # the scale pass reads every K and V row once more
    warmup = max(3, args.warmup)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        if computed:
            k_s, v_s = kv_cache.compute_kv_scales(key, value, slots)
            kv_cache.write_kv_cache(key, value, kc, vc, slots, k_s, v_s)
        else:
            kv_cache.write_kv_cache(key, value, kc, vc, slots, ks, vs)

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
    # the kernel alone: one event pair per call, calls queued back to back (one kernel per call)
    n_timed = min(args.steps, 50)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_timed)]
    for a, b in pairs:
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    kernel_ms = sum(a.elapsed_time(b) for a, b in pairs) / n_timed
    # end to end: the step's rows and slot ids come from pinned host memory; the cache is resident device state
    host = dict(key=key.cpu().pin_memory(), value=value.cpu().pin_memory(), slots=slots.cpu().pin_memory())
    done = torch.zeros(1, dtype=torch.int64).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())

    def e2e_step():
        key.copy_(host["key"], non_blocking=True)
        value.copy_(host["value"], non_blocking=True)
        slots.copy_(host["slots"], non_blocking=True)
        step()
        done.copy_(slots[-1:], non_blocking=True)   # the write returns nothing: read back one word as the completion
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(1, min(args.steps, 10))
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    stats = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = stats.tolist()
    if rank == 0:
        peaks = measured_peaks()
        achieved = work / (kernel_ms * 1e-3) / 1e9
        line = dict(
            metric=kind["metric"], value=work * world * args.steps / (elapsed_ms * 1e-3) / 1e9, unit="GB/s",
            n_gpus=world, steps=args.steps, warmup=warmup, ms_per_step=elapsed_ms / args.steps,
            higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16->e4m3" if spec["fp8"] else "bf16",
            data="synthetic",
            config=dict(workload=args.workload, new_tokens=spec["tokens"], num_kv_heads=spec["hkv"],
                        head_dim=spec["d"], page_size=spec["page"], cache="interleaved K|V pool, random page order",
                        sharding="one step per rank, no collective",
                        l2="rows read + written per step (0.8 - 1.07 GB) >> 126 MB L2",
                        algorithmic_work_per_step_rank0=work),
            roofline=dict(bound="hbm", achieved=achieved, peak=peaks["hbm"], unit="GB/s", frac=achieved / peaks["hbm"],
                          traffic=NCU_TRAFFIC_RATIO.get(args.workload, 1.0) * work, peak_source=peaks["source"],
                          kernel="atrex_sm100_kv_amax_kernel + atrex_sm100_kv_write_kernel" if computed
                          else "atrex_sm100_kv_write_kernel", kernel_ms=kernel_ms,
                          frac_of_nominal_8tbs=achieved / 8000.0),
            e2e=dict(value=work * world / (e2e_ms * 1e-3) / 1e9, unit="GB/s", h2d_bytes_per_step=h2d,
                     d2h_bytes_per_step=8, steps=e2e_steps,
                     note="the step's K/V rows and slot ids copied from pinned host memory each step (PCIe-bound); "
                          "the caches are resident device state"),
            gpu_launches=args.steps * (3 if computed else 1), clocks=dict(sm_mhz=clocks["sm_mhz"], sm_max_mhz=clocks["sm_max_mhz"],
                                                 reasons=clocks["reasons"]),
            device_status=runtime.check_device_status(device),
        )
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = kv_write_cpu(spec, 1729, 10.0)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
# Measurement of one attention workload
# ---------------------------------------------------------------------------------------------------------------
SUB_RESULTS = ("decode_q4_window", "prefill_fp8_hd256", "prefill_hd128", "prefill_sharded")
SUB_BUDGET_S = 8.0      # device time one sub-result's timed samples may take: steps per sample are cut to fit


def shard_requests(spec, world, rank, base_seed=1729):
    """The requests rank ``rank`` of ``world`` serves, and the per-rank loads of the partition.

    "strong" workloads are one fixed request set; "weak" ones pool the batches of all ranks (seed
    ``base_seed + 1000 * r`` for rank r, so the one-GPU run is the plain seeded batch).  The pool is dealt by cost,
    longest first (``sharding.partition_requests``); cost = the request's algorithmic work.  Pure host arithmetic:
    every rank derives the same partition without communicating."""
    from atrex.src.nvidia.flash_attn.sm100 import sharding

    if spec["scaling"] == "strong":
        all_q, all_kv = draw_lengths(spec, base_seed)
    else:
        all_q, all_kv = [], []
        for r in range(world):
            q, kv = draw_lengths(spec, base_seed + 1000 * r)
            all_q += q
            all_kv += kv
    costs = [work_units(spec, [a], [b]) for a, b in zip(all_q, all_kv)]
    shards = sharding.partition_requests(costs, world)
    loads = sharding.shard_loads(costs, shards)
    mine = shards[rank]
    return [all_q[i] for i in mine], [all_kv[i] for i in mine], loads


class Job:
    """Rank, devices and the modules a measurement needs."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.args, self.torch, self.dist = args, torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.device = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def reduce(self, values, op="max"):
        t = self.torch.tensor(list(values), dtype=self.torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.SUM)
        return t.tolist()

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def fp8_gemm_yardstick(torch, device, seconds=2.0):
    """E4M3 x E4M3 -> BF16 GEMM rate of the vendor library (torch._scaled_mm, 8192^3): best single call and the
    rate of a loop of ``seconds``.  A yardstick for the FP8 roofline fraction only; nothing on the attention path
    calls it."""
    n = 8192
    try:
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=device)
        run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            run()
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e))
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        count, t0 = 0, time.perf_counter()
        s.record()
        while time.perf_counter() - t0 < seconds:
            for _ in range(20):
                run()
            count += 20
            torch.cuda.synchronize()
        e.record()
        torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        return dict(burst=flops / (best * 1e-3) / 1e12, sustained=flops * count / (s.elapsed_time(e) * 1e-3) / 1e12,
                    how=f"torch._scaled_mm E4M3 {n}^3 -> BF16: best of 10 calls, and a {seconds:.0f} s loop")
    except Exception as exc:  # the library call is optional evidence, never a dependency
        return dict(burst=None, sustained=None, how=f"torch._scaled_mm unavailable: {type(exc).__name__}: {exc}"[:200])


def measure_attention(job, name, spec, steps, warmup, samples, *, num_splits=0, route_name="auto", budget_s=None,
                      with_cpu_baseline=False):
    """Time one attention workload on this job's ranks.  Returns the result dict on rank 0, None elsewhere."""
    torch, dist, device, rank, world = job.torch, job.dist, job.device, job.rank, job.world
    import atrex
    from atrex.src.nvidia.flash_attn.sm100 import launch, runtime, sharding

    kind = KIND[spec["kind"]]
    route = dict(auto=runtime.ROUTE_AUTO, mma=runtime.ROUTE_MMA, umma=runtime.ROUTE_UMMA)[route_name]
    launch.DEFAULT_ROUTE = route
    variant = spec.get("variant")
    seed = 1729 + 1000 * rank
    work_spec, extra_call = spec, {}
    if variant is None:
        q_lens, kv_lens, loads = shard_requests(spec, world, rank)
        case_kv = kv_lens
        sharding_note = ("one request pool (the N ranks' batches), dealt by cost longest-first, no collective"
                         if spec["scaling"] == "weak" else
                         "one fixed request set, dealt by cost longest-first, no collective")
    else:
        q_lens, kv_lens = draw_lengths(spec, 1729)          # every rank serves every request
        loads = None
        if variant == "cp":
            case_kv = [len(range(rank, n, world)) for n in kv_lens]     # keys rank, rank + W, ... of each request
            sharding_note = "keys of every request dealt round-robin to the ranks; (O, LSE) all-gathered and merged"
        else:
            case_kv = kv_lens
            if spec["hkv"] % world:
                raise SystemExit(f"{name}: {spec['hkv']} KV heads do not divide over {world} ranks")
            work_spec = dict(spec, hq=spec["hq"] // world, hkv=spec["hkv"] // world)
            sharding_note = "KV heads (and their query heads) split over the ranks; O all-gathered"
            seed = 1729
    case, host = build_device_case(spec, q_lens, case_kv, seed, device)
    case["num_splits"] = num_splits
    if variant == "cp" and world > 1:
        extra_call = dict(cp_world_size=world, cp_rank=rank,
                          cp_tot_seqused_k=torch.tensor(kv_lens, dtype=torch.int32, device=device))
        case.update(extra_call)
    if variant == "headsplit" and world > 1:
        qh, kh = sharding.split_heads(spec["hq"], spec["hkv"], world, rank)
        case["q"] = case["q"][:, qh].contiguous()
        case["k"], case["v"] = case["k"][:, :, kh], case["v"][:, :, kh]       # views: strides unchanged
        case["out"] = torch.empty(case["q"].shape, dtype=torch.bfloat16, device=device)
        host["q"] = case["q"].cpu().pin_memory()
    my_work = work_units(work_spec, q_lens, case_kv)

    exchange = None
    if variant == "cp" and world > 1 and job.args.cp_exchange == "fused":
        exchange = sharding.ContextParallelExchange(case["q"].shape[0], spec["hq"], spec["d"], device)
        sharding_note += "; exchange + merge = one kernel over peer loads (symmetric memory)"
    elif variant == "cp":
        sharding_note += "; exchange = two NCCL all-gathers, then the merge kernel"

    def step(case=case):
        if exchange is not None:
            case["out"] = exchange.out_buffer(case["q"].shape[0])
            result = atrex.flash_attn_varlen_func(**case)
            return exchange.merge(case["q"].shape[0], result[1])[0]
        result = atrex.flash_attn_varlen_func(**case)
        if variant == "cp":
            return sharding.gather_context_parallel(result[0], result[1], world)[0]
        out = result[0] if isinstance(result, tuple) else result
        if variant == "headsplit":
            return sharding.gather_heads(out, world)
        return out

    # ---------------- steps per sample: all of --steps unless a time budget asks for fewer ----------------
    warmup = max(3, warmup)
    step()
    job.barrier()
    if budget_s is not None:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        one_ms = job.reduce([a.elapsed_time(b)])[0]
        fit = int(budget_s * 1e3 / max(one_ms, 1e-3) / samples)
        if fit < 1:
            samples = max(3, min(samples, int(budget_s * 1e3 / max(one_ms, 1e-3))))
            fit = 1
        steps = max(1, min(steps, fit))
        warmup = max(3, min(warmup, steps))

    # ---------------- inputs resident: R samples of exactly `steps` steps ----------------
    for _ in range(warmup):
        step()
    job.barrier()
    sampler = ClockSampler(physical_gpu_index(job.local))
    sampler.start()
    sample_ms = []
    for _ in range(samples):
        job.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            step()
        stop.record()
        job.barrier()
        sample_ms.append(start.elapsed_time(stop))
    clocks = sampler.stop()

    # ---------------- dominant kernel alone (events recorded by the launcher around it) ----------------
    window = spec["window"] or (-1, -1)
    lse_buf = (torch.empty((case["q"].shape[1], case["q"].shape[0]), dtype=torch.float32, device=device)
               if spec["lse"] else None)
    params = runtime.build_params(case["q"], case["k"], case["v"], case["out"], lse_buf, case["cu_seqlens_q"], None,
                                  case["seqused_k"], case["block_table"], case.get("q_descale"), case.get("k_descale"),
                                  case.get("v_descale"), case.get("s_aux"), None, case["max_seqlen_q"],
                                  case["max_seqlen_k"], case["softmax_scale"], 0.0, True, window[0], window[1],
                                  num_splits, route, extra_call.get("cp_world_size", 1), extra_call.get("cp_rank", 0),
                                  extra_call.get("cp_tot_seqused_k"))
    info = runtime.plan(params)
    workspace = torch.empty(max(1, info.workspace_bytes), dtype=torch.uint8, device=device)
    lib = runtime.load_library()
    stream = torch.cuda.current_stream().cuda_stream
    # Calls are queued back to back, each with its own event pair, so that an event is recorded when the previous
    # call's last kernel retires and the attention kernel starts right behind it (no idle-GPU launch latency inside
    # the measured interval).
    n_timed = max(3, min(steps * samples, 50))
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_timed)]
    for a, b in pairs:
        a.record()
        b.record()
    torch.cuda.synchronize()
    # The GPU has idled since the timed steps (the clock sampler is joined, the events above are created): ~30 ms of
    # untimed calls come first, so that the timed launches do not run while the clocks ramp up again.
    lead = max(3, min(200, int(30.0 * steps / max(statistics.median(sample_ms), 1e-3)) + 1))
    for i in range(lead + n_timed):
        a, b = pairs[max(i - lead, 0)]
        params.profile_event_begin, params.profile_event_end = a.cuda_event, b.cuda_event
        runtime.raise_for_status(lib.atrex_fa_sm100_forward(ctypes.byref(params), workspace.data_ptr(),
                                                             workspace.numel(), stream))
    torch.cuda.synchronize()
    kernel_ms = sorted(a.elapsed_time(b) for a, b in pairs)
    kernel_ms_avg = sum(kernel_ms) / len(kernel_ms)

    # ---------------- end to end: host inputs in, host result out ----------------
    skip_e2e = case["q"].numel() * case["q"].element_size() > E2E_MAX_BYTES
    # The step's inputs travel as ONE pinned buffer and one copy (each at a 256-byte aligned offset), the way a
    # serving loop stages its per-step tensors; the call reads views of the device copy.
    offsets, cursor = {}, 0
    for key, src in host.items():
        offsets[key] = cursor
        cursor += (src.numel() * src.element_size() + 255) // 256 * 256
    staged_host = torch.empty(max(cursor, 1), dtype=torch.uint8).pin_memory()
    staged_dev = torch.empty(max(cursor, 1), dtype=torch.uint8, device=device)
    e2e_case = dict(case)
    for key, src in host.items():
        nbytes = src.numel() * src.element_size()
        staged_host[offsets[key]: offsets[key] + nbytes].copy_(src.contiguous().view(torch.uint8).reshape(-1))
        if not skip_e2e or key != "q":
            e2e_case[key] = staged_dev[offsets[key]: offsets[key] + nbytes].view(src.dtype).view(src.shape)
    out_shape = (1,) if skip_e2e else ((case["q"].shape[0], spec["hq"], spec["d"]) if variant == "headsplit"
                                       else tuple(case["out"].shape))
    out_host = torch.empty(out_shape, dtype=torch.bfloat16).pin_memory()
    h2d = staged_host.numel()
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step(sync=True):
        staged_dev.copy_(staged_host, non_blocking=True)
        out_host.copy_(step(e2e_case), non_blocking=True)
        if sync:
            torch.cuda.current_stream().synchronize()

    e2e_steps = steps if spec["kind"] == "decode" else max(1, min(steps, 5))
    e2e_samples = max(3, min(samples, 5))
    e2e_sample_ms, e2e_pipelined_ms = [float("nan")], float("nan")
    if not skip_e2e:
        for _ in range(3):
            e2e_step()
        e2e_sample_ms = []
        for _ in range(e2e_samples):
            job.barrier()
            t0 = time.perf_counter()
            s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s2.record()
            for _ in range(e2e_steps):
                e2e_step()
            e2.record()
            job.barrier()
            # every step ends with a host-side stream synchronise: wall clock and device events bracket the same work
            e2e_sample_ms.append(max(s2.elapsed_time(e2), (time.perf_counter() - t0) * 1e3) / e2e_steps)
        # the same steps queued without waiting for each result (one synchronise at the end), the way a serving
        # loop issues them: the host's per-call work then overlaps the previous step's kernel
        job.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step(sync=False)
        job.barrier()
        e2e_pipelined_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    # The same step (copy in, the public call, copy out) captured once as a CUDA graph and replayed, waiting for every
    # step's result: how a serving engine issues its decode steps (the reference's decode tests time graph replays
    # too, op_test/nvidia/qsa/test_qsa_sm100.py:454-471).  Every replay re-reads the pinned host buffer.
    e2e_graph_ms = [float("nan")]
    # Single-process runs only: with a process group alive its watchdog thread makes CUDA calls of its own, which a
    # stream capture in the default (global) mode does not tolerate.
    if not skip_e2e and variant is None and spec["kind"] == "decode" and world == 1:
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            e2e_step(sync=False)
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                e2e_step(sync=False)
        torch.cuda.synchronize()
        out_host.zero_()
        graph.replay()
        torch.cuda.synchronize()
        if not torch.equal(out_host, step(e2e_case).cpu()):
            raise SystemExit(f"{name}: the graph replay's result differs from the eager call's")
        e2e_graph_ms = []
        for _ in range(e2e_samples):
            job.barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                graph.replay()
                torch.cuda.current_stream().synchronize()
            e2e_graph_ms.append((time.perf_counter() - t0) * 1e3 / e2e_steps)
            job.barrier()
    status = runtime.check_device_status(device)

    # ---------------- reduce over ranks: per sample the slowest rank counts ----------------
    sample_ms = job.reduce(sample_ms)
    e2e_sample_ms = job.reduce(e2e_sample_ms)
    e2e_pipelined_ms = job.reduce([e2e_pipelined_ms])[0]
    e2e_graph_ms = job.reduce(e2e_graph_ms)
    total = job.reduce([float(my_work)], op="sum")[0]
    if rank != 0:
        return None
    peaks = measured_peaks()
    peak = peaks[kind["bound"]]
    med_ms = statistics.median(sample_ms)
    to_value = lambda ms_total: total * steps / (ms_total * 1e-3) / kind["scale"]  # noqa: E731
    # The event-timed launch includes the gap between the event and the kernel behind it; on some boxes that makes a
    # short kernel come out longer than a whole step (attention + combine).  The kernel cannot take longer than the
    # step that contains it, so the step time then bounds its duration.
    kernel_ms_source = "events around the attention kernel"
    if kernel_ms_avg > med_ms / steps:
        kernel_ms_avg = med_ms / steps
        kernel_ms_source = "whole step (the event-timed launch came out longer than the step that contains it)"
    achieved = my_work / (kernel_ms_avg * 1e-3) / kind["scale"]
    kernel_name = "atrex_sm100_fwd_mma_kernel"
    if info.route == runtime.ROUTE_UMMA:
        kernel_name = "atrex_sm100_fwd_umma_kernel" if info.m_rows == 256 else "atrex_sm100_fwd_umma1_kernel"
    ratio = NCU_TRAFFIC_RATIO.get(name)
    traffic = None if ratio is None else ratio * my_work
    if name in NCU_PREFILL_IO_RATIO:      # Q read, O written, K and V read once (BF16)
        io_bytes = 2 * (2 * sum(q_lens) * spec["hq"] + 2 * sum(case_kv) * spec["hkv"]) * spec["d"]
        traffic, ratio = NCU_PREFILL_IO_RATIO[name] * io_bytes, NCU_PREFILL_IO_RATIO[name]
    roofline = dict(bound=kind["bound"], achieved=achieved, peak=peak, unit=kind["unit"], frac=achieved / peak,
                    traffic=traffic, peak_source=peaks["source"],
                    kernel=kernel_name, kernel_ms=kernel_ms_avg, kernel_ms_min=kernel_ms[0],
                    kernel_ms_max=kernel_ms[-1], kernel_launches_timed=len(kernel_ms),
                    kernel_ms_source=kernel_ms_source)
    if ratio is not None:
        roofline["traffic_note"] = ("bytes per launch: ncu dram read+write of a small case of this kernel, scaled by "
                                    "bytes processed")
    if kind["bound"] == "hbm":
        roofline["frac_of_nominal_8tbs"] = achieved / 8000.0
    else:
        roofline["peak_kind"] = "sustained cuBLAS bf16 (kernel timed inside a long step)"
        roofline["frac_of_burst_peak"] = achieved / peaks["tensor_burst"]
        roofline["frac_of_nominal_2250"] = achieved / 2250.0
        if spec.get("fp8"):
            yard = fp8_gemm_yardstick(torch, device)
            roofline["peak_fp8_measured"] = yard
            roofline["frac_of_nominal_fp8_4500"] = achieved / 4500.0
            if yard["sustained"]:
                roofline["frac_bf16_peak"] = roofline["frac"]
                roofline["peak"], roofline["frac"] = yard["sustained"], achieved / yard["sustained"]
                roofline["frac_of_burst_peak"] = achieved / yard["burst"]
                roofline["peak_kind"] = "sustained E4M3 GEMM of the vendor library (torch._scaled_mm), measured in this run"
            else:
                roofline["note"] = "no FP8 GEMM rate could be measured here: frac is against the measured BF16 rate"
    e2e_med = statistics.median(e2e_sample_ms)
    per_step = info.kernel_launches
    result = dict(
        metric=kind["metric"], value=to_value(med_ms), unit=kind["unit"], n_gpus=world, steps=steps, warmup=warmup,
        samples=len(sample_ms), ms_per_step=med_ms / steps,
        spread=dict(ms_per_step_min=min(sample_ms) / steps, ms_per_step_max=max(sample_ms) / steps,
                    value_min=to_value(max(sample_ms)), value_max=to_value(min(sample_ms)),
                    note="median of the samples is reported; each sample = `steps` calls, slowest rank"),
        higher_is_better=True, scaling=spec["scaling"], vs_baseline=None,
        dtype="fp8_e4m3" if spec.get("fp8") else "bf16", data="synthetic",
        config=dict(workload=name, requests_on_rank0=len(q_lens), batch=spec["batch"], num_q_heads=spec["hq"],
                    num_kv_heads=spec["hkv"], head_dim=spec["d"], page_size=spec["page"], q_tokens_rank0=sum(q_lens),
                    kv_tokens_rank0=sum(case_kv), max_kv_len=max(case_kv), num_splits=info.num_splits,
                    route=route_name, sharding=sharding_note,
                    rank_loads_max_over_mean=(None if not loads else max(loads) / (sum(loads) / len(loads))),
                    l2="inputs larger than L2 (K/V + Q touched per step >> 126 MB)",
                    algorithmic_work_per_step_rank0=my_work),
        roofline=roofline,
        e2e=dict(value=None if skip_e2e else total / (e2e_med * 1e-3) / kind["scale"], unit=kind["unit"],
                 h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, steps=0 if skip_e2e else e2e_steps,
                 samples=0 if skip_e2e else len(e2e_sample_ms),
                 value_min=None if skip_e2e else total / (max(e2e_sample_ms) * 1e-3) / kind["scale"],
                 value_max=None if skip_e2e else total / (min(e2e_sample_ms) * 1e-3) / kind["scale"],
                 pipelined_value=None if skip_e2e else total / (e2e_pipelined_ms * 1e-3) / kind["scale"],
                 graph_value=(None if e2e_graph_ms[0] != e2e_graph_ms[0] else
                              total / (statistics.median(e2e_graph_ms) * 1e-3) / kind["scale"]),
                 skipped="Q exceeds the pinned staging limit of this benchmark" if skip_e2e else None,
                 note="per-step inputs (q, cu_seqlens_q, seqused_k, block_table) copied from pinned host memory as one "
                      "staged buffer, O copied back; the paged KV cache is resident device state; `value` waits for "
                      "every step's result before issuing the next, `pipelined_value` queues the same steps and "
                      "waits once, `graph_value` replays the step captured as one CUDA graph and waits for every result"),
        gpu_launches=per_step * steps * len(sample_ms), gpu_launches_per_step=per_step,
        clocks=dict(sm_mhz=clocks["sm_mhz"], sm_max_mhz=clocks["sm_max_mhz"], reasons=clocks["reasons"]),
        device_status=status,
    )
    if with_cpu_baseline:
        result["cpu_baseline"], _ = cpu_baseline(spec, q_lens, kv_lens, seed)
    return result


def measure_host_path(job, spec):
    """Host time of one public call on rank 0: enqueue-only loop (nothing waits for the GPU inside it), best of 5
    runs of 200 calls, and the same for the eligibility check alone (the full validation, which a repeated call
    signature skips)."""
    torch = job.torch
    import atrex

    if job.rank != 0:
        return None
    q_lens, kv_lens = draw_lengths(spec, 1729)
    case, _ = build_device_case(spec, q_lens, kv_lens, 1729, job.device)
    for _ in range(20):
        atrex.flash_attn_varlen_func(**case)
    torch.cuda.synchronize()

    def best_of(fn):
        best = float("inf")
        for _ in range(5):
            t0 = time.perf_counter()
            for _ in range(200):
                fn()
            best = min(best, (time.perf_counter() - t0) / 200 * 1e6)
            torch.cuda.synchronize()
        return best

    call_us = best_of(lambda: atrex.flash_attn_varlen_func(**case))
    check_us = best_of(lambda: atrex.can_use_flash_attn_varlen_func(**case))
    return dict(host_us_per_call=call_us, full_validation_us=check_us,
                how="200 public calls enqueued back to back without waiting for the GPU, best of 5 runs; "
                    "full_validation_us = can_use_flash_attn_varlen_func alone (every check, no launch)")


def qsa_inputs(spec, seed, device, torch):
    """Rows of `requests` requests, each with its own paged cache of `tokens` tokens; decode rows sit at the end of
    their request, prefill rows are the request's last `rows` positions; every row lists 512 distinct blocks drawn
    from the blocks it can see."""
    rows, requests, tokens, page = spec["rows"], spec["requests"], spec["tokens"], spec["page"]
    hq, hkv = spec["hq"], spec["hkv"]
    g = torch.Generator(device=device).manual_seed(seed)
    width = -(-tokens // page)
    pages = requests * width
    dtype = torch.float8_e4m3fn if spec["fp8"] else torch.bfloat16
    k = (torch.randn((pages, page, hkv, 256), generator=g, device=device) * 0.5).to(dtype)
    v = torch.randn((pages, page, hkv, 256), generator=g, device=device).to(dtype)
    q = (torch.randn((rows, hq, 256), generator=g, device=device) * 0.5).to(dtype)
    gate = torch.randn((rows, hq, 256), generator=g, device=device).bfloat16()
    table = torch.randperm(pages, generator=g, device=device).int().reshape(requests, width)
    per = rows // requests
    req = torch.arange(requests, device=device, dtype=torch.int32).repeat_interleave(per)
    pos = (tokens - per + torch.arange(rows, device=device) % per).long()
    rank = torch.rand((rows, (tokens + 3) // 4), generator=g, device=device)
    rank.masked_fill_(torch.arange(rank.shape[1], device=device)[None, :] >= ((pos + 1) // 4)[:, None], 2.0)
    ids = rank.argsort(dim=1)[:, :512].int().contiguous()
    del rank
    return dict(q=q, k_cache=k, v_cache=v, indexer_block_ids=ids, query_positions=pos, block_table=table,
                token_to_req=req, use_prefill_config=per > 4, output_gate=gate,
                out=torch.empty((rows, hq, 256), dtype=torch.bfloat16, device=device))


def qsa_work_bytes(spec, ids, pos):
    """Bytes of the K and V rows the rows gather (four-token blocks and the unfinished block), Q, gate and out, and
    the index data read per row."""
    visible = pos + 1
    gathered = int((np.minimum(visible // 4, 512) * 4 + visible % 4).sum())
    es = 1 if spec["fp8"] else 2
    rows = len(pos)
    return gathered * spec["hkv"] * 256 * 2 * es + rows * spec["hq"] * 256 * (es + 2 + 2) + rows * (512 * 4 + 12)


def run_qsa(args, spec, rank, world, local):
    """Compact sparse attention workloads: same JSON contract; one or two kernels per call."""
    import torch
    import torch.distributed as dist
    import atrex
    from atrex.src.nvidia.flash_attn.sm100 import runtime
    from atrex.src.nvidia.qsa.sm100 import runtime as qsa_runtime

    kind = KIND["qsa"]
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    runtime.prewarm(device)
    data = qsa_inputs(spec, 1729 + 1000 * rank, device, torch)
    kwargs = dict(sm_scale=256 ** -0.5 * 0.5, v_scale=1.25) if spec["fp8"] else {}
    work = qsa_work_bytes(spec, None, data["query_positions"].cpu().numpy())
    info = qsa_runtime.plan(qsa_runtime.build_params(
        data["q"], data["k_cache"], data["v_cache"], data["indexer_block_ids"], data["query_positions"],
        data["block_table"], data["token_to_req"], data["output_gate"], data["out"],
        kwargs.get("sm_scale", 256 ** -0.5), kwargs.get("v_scale", 1.0)))
    warmup, steps, samples = max(3, args.warmup), max(1, args.steps), max(1, args.samples)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        if args.num_splits:      # development knob: the public call has no split argument
            return qsa_runtime.forward(data["q"], data["k_cache"], data["v_cache"], data["indexer_block_ids"],
                                       data["query_positions"], data["block_table"], data["token_to_req"], False,
                                       data["output_gate"], data["out"], sm_scale=kwargs.get("sm_scale", 256 ** -0.5),
                                       v_scale=kwargs.get("v_scale", 1.0), num_splits=args.num_splits)
        return atrex.qsa_compact(**data, **kwargs)

    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    sample_ms = []
    for _ in range(samples):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            step()
        stop.record()
        barrier()
        sample_ms.append(start.elapsed_time(stop))
    clocks = sampler.stop()
    # The device time of a call alone: ten calls captured in one CUDA graph (the reference times its decode paths by
    # graph replay too, op_test/nvidia/qsa/test_qsa_sm100.py:454-471), replayed back to back, so that the host's
    # per-call work - longer than the kernels for the decode shapes - is outside the interval.
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(10):
                step()
    torch.cuda.synchronize()
    call_ms = []
    for _ in range(3 + max(3, min(samples, 7))):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        call_ms.append(a.elapsed_time(b) / 10)
    call_ms = sorted(call_ms[3:])
    # end to end: the step's own tensors (Q, gate, block ids, positions, request ids) come from pinned host memory,
    # the result goes back; caches and page table are resident device state
    names = ("q", "output_gate", "indexer_block_ids", "query_positions", "token_to_req")
    host = {n: (data[n].view(torch.uint8) if data[n].dtype == torch.float8_e4m3fn else data[n]).cpu().pin_memory()
            for n in names}
    dev = {n: (data[n].view(torch.uint8) if data[n].dtype == torch.float8_e4m3fn else data[n]) for n in names}
    out_host = torch.empty(data["out"].shape, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())

    def e2e_step():
        for n in names:
            dev[n].copy_(host[n], non_blocking=True)
        out_host.copy_(step(), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    e2e_ms = []
    for _ in range(max(3, min(samples, 5))):
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            e2e_step()
        barrier()
        e2e_ms.append((time.perf_counter() - t0) * 1e3 / steps)
    stats = torch.tensor(sample_ms + e2e_ms, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    sample_ms, e2e_ms = stats.tolist()[: len(sample_ms)], stats.tolist()[len(sample_ms):]
    if rank == 0:
        peaks = measured_peaks()
        med = statistics.median(sample_ms)
        call = sum(call_ms) / len(call_ms)
        achieved = work / (call * 1e-3) / 1e9
        line = dict(
            metric=kind["metric"], value=work * world * steps / (med * 1e-3) / 1e9, unit="GB/s", n_gpus=world,
            steps=steps, warmup=warmup, samples=len(sample_ms), ms_per_step=med / steps,
            spread=dict(ms_per_step_min=min(sample_ms) / steps, ms_per_step_max=max(sample_ms) / steps),
            higher_is_better=True, scaling="weak", vs_baseline=None, dtype="fp8_e4m3" if spec["fp8"] else "bf16",
            data="synthetic",
            config=dict(workload=args.workload, rows=spec["rows"], requests=spec["requests"],
                        tokens_per_request=spec["tokens"], num_q_heads=spec["hq"], num_kv_heads=spec["hkv"],
                        head_dim=256, page_size=spec["page"], blocks_per_row=512, num_splits=info.num_splits,
                        sharding="one batch per rank, no collective",
                        l2="K/V rows gathered per step (134 MB BF16) spread over a 4.3 GB cache: above the 126 MB L2"
                        if spec["requests"] > 1 else "one request's 32 MB cache: L2-resident gather",
                        algorithmic_work_per_step_rank0=work),
            roofline=dict(bound="hbm", achieved=achieved, peak=peaks["hbm"], unit="GB/s", frac=achieved / peaks["hbm"],
                          traffic=None if args.workload not in NCU_TRAFFIC_RATIO else NCU_TRAFFIC_RATIO[args.workload] * work,
                          peak_source=peaks["source"],
                          kernel="atrex_sm100_qsa_kernel" + (" + atrex_sm100_qsa_combine_kernel" if info.num_splits > 1 else ""),
                          kernel_ms=call, kernel_ms_min=call_ms[0], kernel_ms_max=call_ms[-1],
                          frac_of_nominal_8tbs=achieved / 8000.0,
                          note="kernel_ms is the device time of one whole call (attention kernel and, when split, its "
                               "combine): ten calls in one CUDA graph, replayed"),
            e2e=dict(value=work * world / (statistics.median(e2e_ms) * 1e-3) / 1e9, unit="GB/s", h2d_bytes_per_step=h2d,
                     d2h_bytes_per_step=out_host.numel() * 2, steps=steps, samples=len(e2e_ms),
                     note="Q, gate, block ids, positions and request ids copied from pinned host memory each step, out "
                          "copied back; caches and page table are resident device state"),
            gpu_launches=info.kernel_launches * steps * len(sample_ms), gpu_launches_per_step=info.kernel_launches,
            clocks=dict(sm_mhz=clocks["sm_mhz"], sm_max_mhz=clocks["sm_max_mhz"], reasons=clocks["reasons"]),
            device_status=runtime.check_device_status(device),
        )
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = qsa_cpu(spec, data, kwargs, work)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def qsa_cpu(spec, data, kwargs, work_all):
    """The numpy oracle over the first rows of the step (about 10 s)."""
    from oracle import qsa_oracle

    def host(t):
        return (t.float() if t.is_floating_point() else t).cpu().numpy()

    done, rows, t_total = 0, 0, 0.0
    k, v, table = host(data["k_cache"]), host(data["v_cache"]), host(data["block_table"])
    while rows < spec["rows"] and t_total < 10.0:
        sl = slice(rows, rows + 1)
        t0 = time.perf_counter()
        qsa_oracle.qsa_compact(host(data["q"][sl]), k, v, host(data["indexer_block_ids"][sl]),
                               host(data["query_positions"][sl]), table, host(data["token_to_req"][sl]),
                               host(data["output_gate"][sl]), sm_scale=kwargs.get("sm_scale"),
                               v_scale=kwargs.get("v_scale", 1.0))
        t_total += time.perf_counter() - t0
        rows += 1
    return dict(value=work_all * rows / spec["rows"] / t_total / 1e9, unit="GB/s", cores=cpu_threads(), kind="port",
                sample=f"first {rows} of {spec['rows']} rows of the step, {t_total:.1f} s")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--samples", type=int, default=7, help="timed samples of --steps calls each (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_q1", choices=sorted(WORKLOADS))
    ap.add_argument("--num-splits", type=int, default=0)
    ap.add_argument("--route", default="auto", choices=["auto", "mma", "umma"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cp-exchange", default="fused", choices=["fused", "nccl"],
                    help="decode_cp: exchange + merge as one kernel over peer memory, or NCCL all-gathers + merge")
    ap.add_argument("--sub-results", default=None,
                    help="comma-separated workloads measured after the main one and reported under sub_results "
                         "(default: the other configurations of the metric when the workload is decode_q1; 'none')")
    args = ap.parse_args()
    spec = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, spec, rank, world)
        return
    if spec["kind"] == "kv_write":
        run_kv_write(args, spec, rank, world, local)
        return
    if spec["kind"] == "qsa":
        run_qsa(args, spec, rank, world, local)
        return

    job = Job(args)
    from atrex.src.nvidia.flash_attn.sm100 import runtime

    runtime.prewarm(job.device)
    samples = max(1, args.samples)
    line = measure_attention(job, args.workload, spec, max(1, args.steps), args.warmup, samples,
                             num_splits=args.num_splits, route_name=args.route,
                             with_cpu_baseline=job.world == 1 and not args.no_cpu_baseline)
    if args.sub_results is None:
        subs = SUB_RESULTS if args.workload == "decode_q1" else ()
    else:
        subs = tuple(n for n in args.sub_results.split(",") if n and n != "none")
    sub_results = {}
    for name in subs:
        job.torch.cuda.empty_cache()
        try:
            sub = measure_attention(job, name, WORKLOADS[name], max(1, args.steps), args.warmup, samples,
                                    budget_s=SUB_BUDGET_S)
        except Exception as exc:  # noqa: BLE001 - a failed sub-result must not lose the main line
            sub = dict(error=f"{type(exc).__name__}: {exc}"[:300])
        if job.rank == 0:
            sub_results[name] = sub
    if subs and job.rank == 0:
        job.torch.cuda.empty_cache()
        try:
            sub_results["host_path"] = measure_host_path(job, spec)
        except Exception as exc:  # noqa: BLE001
            sub_results["host_path"] = dict(error=f"{type(exc).__name__}: {exc}"[:300])
    if job.rank == 0:
        if sub_results:
            line["sub_results"] = sub_results
        print(json.dumps(line))
    job.close()


if __name__ == "__main__":
    main()
