#!/usr/bin/env python
"""Benchmark of the daisy_b200 attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline (the JSON line's metric/value): windowed causal prefill TFLOP/s on
B=8, T=8192, 16 heads x 128, window 2048, bf16 -- one "step" = q/k/v preparation (RMS norm + RoPE)
plus the windowed attention over one synthetic batch.  The same line carries the decode workload
(batch 64, 16 x 128, ring capacity 32768, window 4096: tokens/s and HBM GB/s) and, when built, the KDA
workload and the long-context prefill (B=1, T=65536, window 8192) as sub-objects, each with its own roofline.

Multi-GPU (torchrun, one rank per GPU), no collective on the data path anywhere:
  * the headline prefill (a configuration quoted "on 1 B200") runs as replicas: every rank its own batch of 8
    independent sequences ("scaling": "weak");
  * the decode workload shards its batch of 64 over the ranks (64/32/16/8 rows per GPU), the long-context
    prefill its 16 heads (16/8/4/2 per GPU), the KDA workload its 64 (batch, head) pairs (64/32/16/8 per GPU).
    These are strong-scaling runs of ONE global problem: rank 0 also runs the whole problem alone, so each
    sub-object carries T(1), T(N) and strong_efficiency = T(1) / (N * T(N)); an NCCL all-gather after the
    timed region reassembles the shard outputs, which must equal that single-GPU result bit for bit.

`--impl reference` times the CPU oracle (the fp32 restatement of the reference's PyTorch path) on a
bounded sample of the same workload with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import threading
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PREFILL_C2 = dict(B=8, T=8192, H=16, D=128, window=2048)
PREFILL_C4 = dict(B=1, T=65536, H=16, D=128, window=8192)
DECODE_C3 = dict(B=64, H=16, D=128, cap=32768, window=4096, steps=256)
KDA_C5 = dict(B=4, T=16384, H=16, K=128, V=128, chunk=64)
# reduced copies of the same kernels for profiler captures (inputs still larger than L2, < 3 GB resident)
PREFILL_SMALL = dict(B=2, T=8192, H=16, D=128, window=2048)
DECODE_SMALL = dict(B=4, H=16, D=128, cap=32768, window=4096, steps=4)
KDA_SMALL = dict(B=1, T=8192, H=16, K=128, V=128, chunk=64)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, transcribed from the ncu captures summarised under
# profiles/ (reduced workloads of the same kernels; traffic grows in proportion to the number of independent
# sequences).  NOT measured by this run: each entry names the summary and the source revision it was captured at,
# and goes stale when that kernel changes.
NCU_TRAFFIC = {
    "prefill_per_batch_row": {"bytes": 1077.9e6 / 8, "profile": "profiles/swa_prefill_kernel__prefill_small.md",
                              "captured_at": "813cf57"},
    "decode_per_batch_row": {"bytes": 137.3e6 / 4, "profile": "profiles/swa_decode_partial_kernel__decode_small.md",
                             "captured_at": "c27d954"},
    "kda_per_token_head": {"bytes": 526.8e6 / 131072, "profile": "profiles/kda_intra_kernel__kda_small.md + profiles/kda_state_kernel__kda_small.md",
                           "captured_at": "601341c"},
}
ROPE_BASE = 10000.0     # the benchmark configs name base 10000 (the module default is 1024, half-truncated)


# ----------------------------------------------------------------------------- helpers

def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), which="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, which="fallback")


class ClockSampler:
    """SM clock and throttle reasons sampled WHILE the timed region runs: NVML from a thread every ~2 ms (the
    timed regions here last tens of milliseconds, too short for `nvidia-smi -lms`), else `nvidia-smi -lms 100`.
    Read-only queries; nothing is set."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.thread = index, None, None
        self.samples, self.reason_bits, self.power = [], 0, []
        self._stop = threading.Event()
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            # NVML numbers devices like nvidia-smi; CUDA_VISIBLE_DEVICES remaps torch's index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if vis:
                ids = [x.strip() for x in vis.split(",") if x.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def _poll(self):
        n = self.nvml
        while not self._stop.is_set():
            try:
                self.samples.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                self.reason_bits |= int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                self.power.append(n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
            except Exception:
                break
            time.sleep(0.002)

    def start(self):
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            n = self.nvml
            names = (("hw_slowdown", "nvmlClocksEventReasonHwSlowdown"), ("hw_thermal_slowdown", "nvmlClocksEventReasonHwThermalSlowdown"),
                     ("sw_thermal_slowdown", "nvmlClocksEventReasonSwThermalSlowdown"), ("sw_power_cap", "nvmlClocksEventReasonSwPowerCap"))
            reasons = sorted(k for k, attr in names if self.reason_bits & int(getattr(n, attr, 0)))
            return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                    "sm_min_mhz": min(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                    "power_w_max": max(self.power) if self.power else None, "reasons": reasons,
                    "samples": len(self.samples), "source": "nvml, 2 ms period, during the timed region"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [x for x in sm if x > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi -lms 100"}


def shard_bounds(n: int, world: int, rank: int):
    """Contiguous split of n independent units (batch rows, heads, batch x heads) over the ranks."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def dist_env():
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    return ws, int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def rope_full(D, T, device):
    """Full (untruncated) cos/sin tables [T, D/2] fp32, frequencies (1/base)**linspace(0, 1, D/2)."""
    freq = (1.0 / ROPE_BASE) ** torch.linspace(0, 1, steps=D // 2, dtype=torch.float32)
    theta = torch.arange(T, dtype=torch.float32)[:, None] * freq[None, :]
    return theta.cos().to(device), theta.sin().to(device)


L2_BYTES = 126 << 20
_flush_buf = {}


def l2_flush_buffer(dev):
    """256 MiB scratch whose rewrite between timed steps evicts the 126 MB L2 (used when a step's own inputs are not
    larger than L2, e.g. the per-GPU shards of the strong-scaling runs)."""
    key = dev.index
    if key not in _flush_buf:
        _flush_buf[key] = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    return _flush_buf[key]


def timed_steps(step, steps, warmup, dist, flush=None):
    """W warm-up steps, then K steps between barrier+synchronize on both sides; device time by CUDA
    events on the launching stream; MAX over ranks.  With `flush` (a buffer larger than L2) every step is
    bracketed by its own pair of events and the buffer is rewritten between steps, outside the events."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    else:
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in ev:
            flush.zero_()
            a.record(); step(); b.record()
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in ev)
    if dist is not None:
        dist.barrier()
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def timed_region(fn, dist):
    """One call of `fn` (which enqueues a whole loop of steps) between barrier + synchronize on both sides;
    device time by CUDA events on the launching stream; MAX over ranks."""
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def unit_shard(B: int, H: int, world: int, rank: int):
    """Shard the B x H independent (batch, head) pairs of one problem over the ranks: whole batch rows while the
    per-rank share is a multiple of H, else a head range of one batch row.  Returns (b_lo, b_hi, h_lo, h_hi)."""
    n = B * H
    if n % world == 0:
        per = n // world
        if per % H == 0:
            return rank * per // H, (rank + 1) * per // H, 0, H
        if H % per == 0:
            u = rank * per
            return u // H, u // H + 1, u % H, u % H + per
    if B < world:
        raise SystemExit(f"cannot shard {B} x {H} (batch, head) pairs evenly over {world} ranks")
    lo, hi = shard_bounds(B, world, rank)
    return lo, hi, 0, H


def strong_summary(t1_ms, tn_ms, world, limiter=None):
    """Strong scaling of one global problem: T(1) is rank 0 running the whole problem alone in this same run.
    ``limiter``: what bounds the efficiency of this workload when it falls below 0.9 (named in the record then)."""
    eff = (t1_ms / (world * tn_ms)) if tn_ms else None
    out = {"t1_ms": t1_ms, "tn_ms": tn_ms, "strong_efficiency": eff}
    if limiter and eff is not None and eff < 0.9:
        out["limiter"] = limiter
    return out


# ----------------------------------------------------------------------------- our arm: prefill

def prefill_inputs(cfg, seed, dev):
    B, T, H, D = cfg["B"], cfg["T"], cfg["H"], cfg["D"]
    g = torch.Generator(device=dev).manual_seed(seed)
    return tuple(torch.randn(B, T, H, D, device=dev, generator=g).bfloat16() for _ in range(3))


def sustained_prefill(step, flops, peaks, dev, seconds=2.0):
    """The same step looped for >= `seconds` so that the power-capped clock settles: TFLOP/s against the measured
    SUSTAINED cuBLAS rate, NVML clock samples (read only), and time x median SM MHz (a clock-normalised figure
    that can be compared between runs).  Rank-local, no barrier."""
    n = 50
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(dev.index or 0)
    torch.cuda.synchronize()
    sampler.start()
    t_begin, total_ms, total_steps, last = time.perf_counter(), 0.0, 0, None
    while time.perf_counter() - t_begin < seconds:
        e0.record()
        for _ in range(n):
            step()
        e1.record()
        torch.cuda.synchronize()
        last = e0.elapsed_time(e1) / n
        total_ms += last * n
        total_steps += n
    clocks = sampler.stop()
    tf = flops / (last * 1e-3) / 1e12                        # the last block: the settled clock
    mhz = clocks.get("sm_mhz")
    return {"seconds": total_ms / 1e3, "steps": total_steps, "ms_per_step_settled": last, "tflops_settled": tf,
            "ms_per_step_mean": total_ms / total_steps, "peak_sustained": peaks["bf16_tflops_sustained"],
            "frac_of_sustained_peak": tf / peaks["bf16_tflops_sustained"], "clocks": clocks,
            "ms_x_mhz": (last * mhz) if mhz else None,
            "note": "TFLOP/s of the last 50-step block of a loop that ran this long; peak = cuBLAS bf16 looped for seconds"}


def run_prefill(cfg, steps, warmup, dist, rank, world, peaks, name, lean=False, shard_heads=False, sustained=False):
    """`shard_heads=False`: every rank runs the whole configuration on its own sequences (replicas, weak scaling).
    `shard_heads=True`: ONE global problem, the heads split over the ranks (strided views of the global q, k, v);
    rank 0 also runs all heads alone for T(1)."""
    from daisy_b200 import ops, _lib
    from daisy_b200 import accounting as acct
    B, T, H, D, W = cfg["B"], cfg["T"], cfg["H"], cfg["D"], cfg["window"]
    dev = torch.device("cuda", torch.cuda.current_device())
    q, k, v = prefill_inputs(cfg, 1234 + (0 if shard_heads else rank), dev)
    h_lo, h_hi = shard_bounds(H, world, rank) if shard_heads else (0, H)
    if shard_heads and H % world != 0:
        raise SystemExit(f"{name}: {H} heads do not split evenly over {world} ranks")
    Hs = h_hi - h_lo
    qs, ks, vs = q[:, :, h_lo:h_hi], k[:, :, h_lo:h_hi], v[:, :, h_lo:h_hi]
    cos, sin = rope_full(D, T, dev)
    L = _lib.lib()
    ws = torch.empty(L.daisy_b200_swa_prefill_workspace_bytes(B, T, H, D), dtype=torch.uint8, device=dev)
    out = torch.empty(B, T, Hs, D, dtype=torch.bfloat16, device=dev)
    k_out = torch.empty(B, T, Hs, D, dtype=torch.bfloat16, device=dev)
    v_out = torch.empty_like(k_out)
    flops_global = acct.prefill_flops(B, T, H, D, W)
    flops_rank = acct.prefill_flops(B, T, Hs, D, W)
    total_flops = flops_global if shard_heads else world * flops_global

    def step():
        ops.swa_prefill(qs, ks, vs, cos, sin, W, eps=acct.FP32_EPS, workspace=ws, out=out, k_out=k_out, v_out=v_out)

    in_bytes_dev = 3 * qs.numel() * 2
    flush = l2_flush_buffer(dev) if (in_bytes_dev < 2 * L2_BYTES and not lean) else None
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    ms = timed_steps(step, steps, warmup, dist, flush)
    clocks = sampler.stop()
    ops.check_device_status(dev)
    per = ms / steps

    if lean:                                                 # profiler capture: the timed loop only
        return {"name": name, "ms_per_step": per, "tflops": total_flops / (per * 1e-3) / 1e12,
                "clocks": clocks, "launches_per_step": 2, "roofline": None, "e2e": None,
                "config": {"workload": f"{name}: B={B} T={T} H={H} D={D} window={W} (profiler capture case)"}}
    # dominant kernel alone (attention on prepared tensors), CUDA events around each launch
    qp, kp, vp = ops.qkv_prep(qs, ks, vs, cos, sin, acct.FP32_EPS)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    out_k = torch.empty_like(out)
    for _ in range(warmup):
        ops.swa_attend(qp, kp, vp, W, out=out_k, bounded_qk=True)      # the kernel the step launches
    torch.cuda.synchronize()
    for a, b in ev:
        a.record(); ops.swa_attend(qp, kp, vp, W, out=out_k, bounded_qk=True); b.record()
    torch.cuda.synchronize()
    k_ms = sum(a.elapsed_time(b) for a, b in ev) / steps
    kernel_same = bool(torch.equal(out_k, out))
    del qp, kp, vp, out_k

    # end to end through the public host-buffer call: pinned host q,k,v in, pinned host result out, every step;
    # batch rows stream through copy-in / kernels / copy-out on three CUDA streams
    from daisy_b200.host_api import HostPrefill
    hq, hk, hv = (x.cpu().pin_memory() for x in (qs, ks, vs))
    hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    host_call = HostPrefill(T, Hs, D, device=dev, rows_per_chunk=1)

    def e2e_step():
        host_call(hq, hk, hv, cos, sin, W, hout, eps=acct.FP32_EPS)

    e2e_steps = max(2, min(steps, 5))
    e2e_ms = timed_steps(e2e_step, e2e_steps, 1, dist)
    torch.cuda.synchronize()
    e2e_same = bool(torch.equal(hout, out.cpu()))             # same inputs -> the host path must reproduce `out`
    in_bytes = 3 * qs.numel() * 2
    out_bytes = out.numel() * 2
    del host_call, hq, hk, hv, hout

    strong = None
    if dist is not None:                                      # reassemble outputs (verification only)
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        if shard_heads and rank == 0:
            full = torch.cat(gathered, dim=2)
        else:
            assert all(torch.isfinite(x[:, :64].float()).all() for x in gathered)
        del gathered
    if shard_heads:
        t1 = per
        same = None
        if world > 1 and rank == 0:                           # the whole problem on one GPU: T(1) and the reference bits
            out1 = torch.empty(B, T, H, D, dtype=torch.bfloat16, device=dev)
            k1, v1 = torch.empty_like(out1), torch.empty_like(out1)

            def step1():
                ops.swa_prefill(q, k, v, cos, sin, W, eps=acct.FP32_EPS, workspace=ws, out=out1, k_out=k1, v_out=v1)

            t1 = timed_steps(step1, steps, warmup, None, flush) / steps
            same = bool(torch.equal(full, out1))
            del out1, k1, v1, full
        items = ((cfg["T"] + 255) // 256) * Hs * cfg["B"]
        strong = strong_summary(t1, per, world, limiter=f"work-item granularity of the persistent grid: {items} items of 256 query rows "
                                                        f"per GPU on {torch.cuda.get_device_properties(dev).multi_processor_count} CTAs = "
                                                        f"{items / torch.cuda.get_device_properties(dev).multi_processor_count:.2f} rounds")
        strong["gathered_equals_single_gpu_result"] = same
    sus = sustained_prefill(step, flops_rank, peaks, dev) if sustained else None
    finite = bool(torch.isfinite(out.float()).all())
    ach = flops_rank / (k_ms * 1e-3) / 1e12
    traffic = None
    if (T, W) == (8192, 2048) and Hs == 16:
        traffic = NCU_TRAFFIC["prefill_per_batch_row"]["bytes"] * B
    res = {
        "name": name, "ms_per_step": per, "tflops": total_flops / (per * 1e-3) / 1e12,
        "clocks": clocks, "finite": finite, "launches_per_step": 2, "steps": steps,
        "roofline": {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": ach / peaks["bf16_tflops"], "traffic": traffic,
                     "traffic_unit": "bytes per launch (ncu dram read+write of one full-size launch; transcribed, see traffic_source)",
                     "traffic_source": NCU_TRAFFIC["prefill_per_batch_row"] if traffic else None,
                     "kernel": "swa_prefill_kernel", "per_rank_heads": Hs,
                     "kernel_ms": k_ms, "kernel_output_equals_step": kernel_same, "peak_source": peaks["which"] + " (burst cuBLAS bf16)",
                     "step_frac_of_burst_peak": flops_rank / (per * 1e-3) / 1e12 / peaks["bf16_tflops"]},
        "e2e": {"value": total_flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                "matches_device_result": e2e_same, "api": "daisy_b200.host_api.HostPrefill"},
        "config": {"workload": f"{name}: B={B} T={T} H={H} D={D} window={W} causal; one step = two launches: RMS-norm q,k,v + RoPE "
                               f"base {int(ROPE_BASE)} (qkv_prep_kernel), then windowed attention (swa_prefill_kernel)",
                   "per_gpu_batch": B, "per_gpu_heads": Hs, "global_batch": B if shard_heads else B * world,
                   "parallelism": (f"heads sharded {H} -> {Hs} per GPU over {world} GPU(s), one global problem, no collective"
                                   if shard_heads else
                                   f"dp{world} replicas: this configuration is quoted on 1 GPU, every rank runs it whole on its own "
                                   "sequences, no collective"),
                   "l2": (f"inputs ({in_bytes_dev >> 20} MiB q,k,v per GPU) exceed L2" if flush is None else
                          f"inputs are {in_bytes_dev >> 20} MiB per GPU: L2 flushed between steps (256 MiB rewrite outside the events)")},
    }
    if strong is not None:
        res["scaling"] = "strong"
        res["strong"] = strong
    if sus is not None:
        res["sustained"] = sus
    return res


def run_prefill_bwd(cfg, steps, warmup, peaks):
    """Backward of the windowed attention at the headline shape (training form): row-wise delta, the
    key-block-stationary dK/dV kernel and the query-block-stationary dQ kernel.  FLOPs are counted as 2.5 x the forward's
    (five products over the admitted pairs against the forward's two; the two recomputed score products of the
    second kernel are not credited)."""
    from daisy_b200 import ops
    from daisy_b200 import accounting as acct
    B, T, H, D, W = cfg["B"], cfg["T"], cfg["H"], cfg["D"], cfg["window"]
    dev = torch.device("cuda", torch.cuda.current_device())
    q, k, v = prefill_inputs(cfg, 77, dev)
    cos, sin = rope_full(D, T, dev)
    qp, kp, vp = ops.qkv_prep(q, k, v, cos, sin, acct.FP32_EPS)
    del q, k, v
    g = torch.Generator(device=dev).manual_seed(78)
    d_o = torch.randn(B, T, H, D, device=dev, generator=g).bfloat16()
    y, lse = ops.swa_attend(qp, kp, vp, W, bounded_qk=True, return_lse=True)
    res = {}

    def step():
        res["g"] = ops.swa_attend_bwd(qp, kp, vp, y, d_o, lse, W)

    ms = timed_steps(step, steps, warmup, None) / steps
    ops.check_device_status(dev)
    first = [t.clone() for t in res["g"]]
    step()
    same = all(torch.equal(a, b) for a, b in zip(first, res["g"]))
    flops = 2.5 * acct.prefill_flops(B, T, H, D, W)
    tf = flops / (ms * 1e-3) / 1e12
    return {"ms_per_step": ms, "tflops": tf, "value": tf, "unit": "TFLOP/s", "steps": steps, "launches_per_step": 3,
            "flops_counted": "2.5 x forward (dP, dV, dK, dQ and one score product over the admitted pairs)",
            "frac_of_burst_peak": tf / peaks["bf16_tflops"], "finite": bool(all(torch.isfinite(t.float()).all() for t in res["g"])),
            "bitwise_reproducible": bool(same),
            "config": {"workload": f"prefill_bwd: B={B} T={T} H={H} D={D} window={W}, gradients w.r.t. prepared q, k, v"}}


# ----------------------------------------------------------------------------- our arm: decode

class DecodeCase:
    """The decode workload for a set of GLOBAL batch rows (a rank's shard, or all rows): ring and per-step inputs are
    seeded per global row, so a shard holds exactly the rows of the global problem it names."""

    def __init__(self, cfg, rows, nq, dev):
        from daisy_b200 import ops, _lib
        from daisy_b200 import accounting as acct
        self.ops, self.acct = ops, acct
        self.B = B = len(rows)
        self.H, self.D, self.cap, self.W = H, D, cap, W = cfg["H"], cfg["D"], cfg["cap"], cfg["window"]
        self.kc = torch.empty(B, H, cap, D, dtype=torch.bfloat16, device=dev)
        self.vc = torch.empty_like(self.kc)
        self.qs, self.ks, self.vs = (torch.empty(nq, B, 1, H, D, dtype=torch.bfloat16, device=dev) for _ in range(3))
        for i, b in enumerate(rows):
            g = torch.Generator(device=dev).manual_seed(4321 + 7919 * int(b))
            self.kc[i] = torch.randn(H, cap, D, device=dev, generator=g).bfloat16()
            self.vc[i] = torch.randn(H, cap, D, device=dev, generator=g).bfloat16()
            for x in (self.qs, self.ks, self.vs):
                x[:, i] = torch.randn(nq, 1, H, D, device=dev, generator=g).bfloat16()
        self.cos, self.sin = rope_full(D, cap + nq + 128, dev)
        self.splits = ops.decode_splits(B, H, W - 1)
        self.ws = torch.empty(_lib.lib().daisy_b200_swa_decode_workspace_bytes(B, H, D, self.splits), dtype=torch.uint8, device=dev)
        self.ws_single = ops.decode_fused_workspace(B, H, D, self.splits, dev)
        self.single_launch = False        # True: the one-launch form of the step (the last split CTA of a row merges)
        self.out = torch.empty(nq, B, 1, H, D, dtype=torch.bfloat16, device=dev)
        self.bytes_per_step = acct.decode_bytes(B, H, D, W - 1)

    def step(self, i):
        """Input row i at position cap + i: the ring is full, so every step wraps and overwrites the oldest slot."""
        t = self.cap + i
        if self.single_launch:
            self.ops.swa_decode_step_fused(self.qs[i], self.ks[i], self.vs[i], self.kc, self.vc, t, self.cap, self.W, self.cos[t],
                                           self.sin[t], eps=self.acct.FP32_EPS, write_ring=True, splits=self.splits,
                                           workspace=self.ws_single, out=self.out[i])
            return
        self.ops.swa_decode_step(self.qs[i], self.ks[i], self.vs[i], self.kc, self.vc, t, self.cap, self.W, self.cos[t], self.sin[t],
                                 eps=self.acct.FP32_EPS, write_ring=True, splits=self.splits, workspace=self.ws, out=self.out[i],
                                 return_new_kv=False)

    def time(self, warmup, nsteps, dist):
        """(ms per step launched from Python, ms per step as ONE CUDA graph of the same nsteps launches pairs).  The graph
        replays the same positions, so it rewrites the same ring slots with the same rows and must reproduce the
        outputs of the plain loop bit for bit."""
        for i in range(warmup):
            self.step(i)
        plain = timed_region(lambda: [self.step(warmup + i) for i in range(nsteps)], dist) / nsteps
        ref = self.out[warmup:warmup + nsteps].clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(nsteps):
                self.step(warmup + i)
        graph.replay()                                              # warm-up replay
        self.out[warmup:warmup + nsteps].zero_()
        graphed = timed_region(graph.replay, dist) / nsteps
        same = bool(torch.equal(self.out[warmup:warmup + nsteps], ref))
        del graph
        return plain, graphed, same

    def time_both(self, warmup, nsteps, dist):
        """The two-launch form (split partials, then the merge) and the single-launch form of the same step, each as a
        plain loop and as one graph.  Returns a dict; 'ms' is the fastest of the four."""
        self.single_launch = False
        p2, g2, same2 = self.time(warmup, nsteps, dist)
        ref = self.out[warmup:warmup + nsteps].clone()
        self.single_launch = True
        p1, g1, same1 = self.time(warmup, nsteps, dist)
        forms_equal = bool(torch.equal(self.out[warmup:warmup + nsteps], ref))
        single = min(p1, g1) < min(p2, g2)
        self.single_launch = single                                  # what later calls of step() use
        return {"ms": min(p1, g1, p2, g2), "plain": p1 if single else p2, "graph": g1 if single else g2,
                "launches_per_step": 1 if single else 2, "graph_same": same1 and same2, "forms_equal": forms_equal,
                "two_launch_ms": min(p2, g2), "single_launch_ms": min(p1, g1)}


def run_decode(cfg, warmup, dist, rank, world, peaks, lean=False, extras=True):
    """The batch is sharded over the ranks (one global problem, strong scaling); rank 0 also runs the whole batch
    alone for T(1) when there is more than one rank."""
    from daisy_b200 import ops
    B, H, D, cap, W, nsteps = cfg["B"], cfg["H"], cfg["D"], cfg["cap"], cfg["window"], cfg["steps"]
    dev = torch.device("cuda", torch.cuda.current_device())
    if B % world != 0:
        raise SystemExit(f"decode: batch {B} does not split evenly over {world} ranks")
    lo, hi = shard_bounds(B, world, rank)
    nq = nsteps + warmup
    ops.status_word(dev)                                     # allocated before any graph capture
    case = DecodeCase(cfg, range(lo, hi), nq, dev)
    Bs = case.B
    if lean:
        plain, graphed, graph_same = case.time(warmup, nsteps, dist)
        tb = None
    else:
        tb = case.time_both(warmup, nsteps, dist)
        plain, graphed, graph_same = tb["plain"], tb["graph"], tb["graph_same"]
    ops.check_device_status(dev)
    per = min(plain, graphed)
    case_bytes = case.bytes_per_step
    gbs = case_bytes / (per * 1e-3) / 1e9
    if lean:
        return {"name": "decode", "ms_per_step": plain, "tokens_per_s": B / (plain * 1e-3), "hbm_gbs": case.bytes_per_step / (plain * 1e-3) / 1e9,
                "steps": nsteps, "launches_per_step": 2, "roofline": None, "e2e": None,
                "config": {"workload": f"decode: batch {B} x {H} x {D}, capacity {cap}, window {W} (profiler capture case)"}}
    # e2e: the step's host inputs (new q,k,v rows) in, the output row back, cache resident
    hq, hk, hv = (x[:8].cpu().pin_memory() for x in (case.qs, case.ks, case.vs))
    hout = torch.empty(case.out[0].shape, dtype=case.out.dtype).pin_memory()
    state = {"i": 0}

    def e2e_step():
        i = state["i"] % 8
        case.qs[i].copy_(hq[i], non_blocking=True); case.ks[i].copy_(hk[i], non_blocking=True); case.vs[i].copy_(hv[i], non_blocking=True)
        case.step(i)
        hout.copy_(case.out[i], non_blocking=True)
        torch.cuda.current_stream().synchronize()           # the token must reach the host before the next one
        state["i"] = i + 1

    e2e_ms = timed_steps(e2e_step, 64, 2, dist)
    first = case.out[warmup].clone()                         # first timed step's output [Bs,1,H,D]
    finite = bool(torch.isfinite(case.out[warmup:].float()).all())
    splits = case.splits
    del case
    torch.cuda.empty_cache()
    strong = strong_summary(per, per, 1)
    strong.update({"t1_plain_ms": plain, "t1_graph_ms": graphed})
    if dist is not None:
        gathered = [torch.empty_like(first) for _ in range(world)]
        dist.all_gather(gathered, first)
        same = None
        if rank == 0:
            full = DecodeCase(cfg, range(B), nq, dev)
            tb1 = full.time_both(warmup, nsteps, None)
            p1, g1 = tb1["plain"], tb1["graph"]
            # the split count follows the per-GPU batch, so the partial sums of a row are merged in a different
            # order than on one GPU: equal up to fp32 reassociation, compared at one bf16 unit of the outputs
            diff = (torch.cat(gathered, 0).float() - full.out[warmup].float()).abs().max().item()
            same = bool(diff <= 2.0 ** -8 * max(1e-3, full.out[warmup].float().abs().max().item()))
            strong = strong_summary(min(p1, g1), per, world,
                                    limiter=f"{case_bytes / 1e6:.0f} MB per step per GPU = {case_bytes / peaks['hbm_gbs'] / 1e3:.0f} us at copy bandwidth: "
                                            "launch gaps and the merge of the splits are what is left of the step")
            strong.update({"t1_plain_ms": p1, "t1_graph_ms": g1, "gathered_max_abs_diff": diff,
                           "splits_single_gpu": full.splits, "splits_per_rank": splits})
            del full
            torch.cuda.empty_cache()
        strong["gathered_equals_single_gpu_result"] = same
    gen = generator_step_latency(H, D, W) if (rank == 0 and extras) else None
    traffic = NCU_TRAFFIC["decode_per_batch_row"]
    return {"name": "decode_c3", "generator_step": gen, "ms_per_step": per, "ms_per_step_plain_launches": plain,
            "ms_per_step_cuda_graph": graphed, "graph_output_equals_plain": graph_same,
            "tokens_per_s": B / (per * 1e-3), "hbm_gbs": world * gbs, "scaling": "strong", "strong": strong,
            "splits": splits, "steps": nsteps, "launches_per_step": tb["launches_per_step"], "finite": finite,
            "forms": {"two_launch_ms": tb["two_launch_ms"], "single_launch_ms": tb["single_launch_ms"],
                      "single_launch_equals_two_launch": tb["forms_equal"]},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": traffic["bytes"] * Bs,
                         "traffic_unit": "bytes per launch (ncu dram read+write on batch 4, scaled by the per-GPU batch; transcribed, see traffic_source)",
                         "traffic_source": traffic, "kernel": "swa_decode_partial_kernel", "per_rank_batch": Bs,
                         "peak_source": peaks["which"] + " (copy bandwidth)", "frac_of_8TBs": gbs / 8000.0},
            "e2e": {"value": B / (e2e_ms / 64 * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": 3 * Bs * H * D * 2, "d2h_bytes_per_step": Bs * H * D * 2},
            "config": {"workload": f"decode_c3: global batch {B} x {H} heads x {D}, ring capacity {cap}, window {W}, "
                                   f"{nsteps} steps from t={cap} (ring wraps every step)", "per_gpu_batch": Bs, "global_batch": B,
                       "parallelism": f"batch sharded {B} -> {Bs} rows per GPU over {world} GPU(s), no collective",
                       "timing": "the fastest of: the two-launch and the single-launch form of the step, each launched step by step from Python and as one CUDA-graph replay of the same loop"}}


def generator_step_latency(H, D, W, layers=4, batch=1, steps=200):
    """The reference's Generator shape (batch 1, `inference/generate.py:76`): one token through `layers` attention
    layers (projections + fused ring decode), issued launch by launch from Python and as one CUDA-graph replay
    with the position in device memory.  Microseconds per token, steady state (full window, wrapped ring)."""
    from daisy_b200 import B200CausalSelfAttention, StepRunner
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    torch.manual_seed(0)
    dim, cap = H * D, 2 * W
    mods = [B200CausalSelfAttention(dim, H, D, max_seq_len=cap + 2 * steps + 64).cuda().eval() for _ in range(layers)]
    res = {}
    for name in ("eager", "graph"):
        run = StepRunner(mods, window=W, cache_capacity=cap, batch=batch)
        run.cache.k.normal_(); run.cache.v.normal_()
        run.cache.t = cap + 1; run.cache.t_dev.fill_(cap + 1)
        x = torch.randn(batch, 1, dim, device="cuda", dtype=torch.bfloat16)
        if name == "graph":
            run.capture_step(batch, dim)
        step = (lambda: run._step_graph(x)) if name == "graph" else (lambda: run._step(x))
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        res[name + "_us_per_token"] = e0.elapsed_time(e1) / steps * 1e3
        del run
    res.update({"layers": layers, "batch": batch, "window": W, "dim": dim})
    return res


def run_projection(B, T, H, D, steps, warmup, lean=False):
    """The GEMMs either side of the attention at the headline shape (the module's forward = fused QKV GEMM +
    attention + output GEMM): the hand-written tcgen05 GEMM whose epilogue applies the norm and RoPE, against
    cuBLAS followed by the separate norm/RoPE pass.  Not part of the headline step (the benchmark configuration
    starts from q, k, v after the projection); reported beside it."""
    import torch.nn.functional as F
    from daisy_b200 import ops
    from daisy_b200 import accounting as acct
    dev = torch.device("cuda", torch.cuda.current_device())
    dim = H * D
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(B, T, dim, device=dev, generator=g).bfloat16()
    w = (torch.randn(4, dim, dim, device=dev, generator=g) * dim ** -0.5).bfloat16()
    wq = w[:3].flatten(end_dim=1)
    cos, sin = rope_full(D, T, dev)

    def ours():
        return ops.qkv_gemm(x, wq, cos, sin, H, acct.FP32_EPS)

    ms = timed_steps(ours, steps, warmup, None) / steps
    flops = 2.0 * B * T * dim * 3 * dim
    res = {"name": "qkv_gemm", "ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12,
           "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": steps,
           "config": {"workload": f"qkv_gemm: x [{B},{T},{dim}] x W_qkv [{3 * dim},{dim}]^T, norm + RoPE in the epilogue"}}
    if lean:
        res.update({"clocks": None, "roofline": None, "e2e": None, "launches_per_step": 1})
        return res

    def lib():
        q, k, v = F.linear(x, wq).view(B, T, 3 * H, D).chunk(3, dim=-2)
        return ops.qkv_prep(q, k, v, cos, sin, acct.FP32_EPS)

    y = torch.randn(B, T, dim, device=dev, generator=g).bfloat16()
    res["cublas_plus_prep_ms"] = timed_steps(lib, steps, warmup, None) / steps
    res["cublas_gemm_alone_ms"] = timed_steps(lambda: F.linear(x, wq), steps, warmup, None) / steps
    o_ms = timed_steps(lambda: ops.gemm_nt(y, w[3]), steps, warmup, None) / steps
    res["out_proj"] = {"ms": o_ms, "tflops": 2.0 * B * T * dim * dim / (o_ms * 1e-3) / 1e12,
                       "cublas_ms": timed_steps(lambda: F.linear(y, w[3]), steps, warmup, None) / steps}
    a, b = ours(), lib()
    res["max_abs_diff_vs_library_path"] = max(float((a[i].float() - b[i].float()).abs().max()) for i in range(3))
    del a, b, y
    # the whole module forward (projection -> attention -> projection): the module's own path (hand-written kernels
    # only) against the same forward composed from torch's GEMMs and the separate norm / RoPE pass
    from daisy_b200 import B200CausalSelfAttention, WindowMask
    os.environ["DISABLE_O_ZERO_INIT"] = "1"
    mod = B200CausalSelfAttention(dim, H, D, max_seq_len=T).cuda().eval()
    mask = WindowMask(PREFILL_C2["window"])

    def library_forward():
        q_, k_, v_ = F.linear(x, mod.qkvo_w[:3].flatten(end_dim=1)).view(B, T, 3 * H, D).chunk(3, dim=-2)
        y_, _, _ = ops.swa_prefill(q_, k_, v_, mod.rotary.cos, mod.rotary.sin, mask.window, mod.attn_scale, mod.norm_eps)
        return F.linear(y_.view(B, T, dim), mod.qkvo_w[3])

    with torch.inference_mode():
        fwd = {"native_ms": timed_steps(lambda: mod(x, None, attn_mask=mask), steps, warmup, None) / steps,
               "library_gemm_ms": timed_steps(library_forward, steps, warmup, None) / steps}
    res["module_forward"] = fwd
    return res


# ----------------------------------------------------------------------------- our arm: KDA

def kda_inputs(cfg, b_lo, b_hi, h_lo, h_hi, dev):
    """The (batch rows, head range) shard of the global KDA problem, contiguous; every global batch row has its own seed."""
    T, H, K = cfg["T"], cfg["H"], cfg["K"]
    qs, ks, vs, gs, bs = [], [], [], [], []
    for b in range(b_lo, b_hi):
        g_ = torch.Generator(device=dev).manual_seed(99 + 7919 * b)
        q, k, v = (torch.randn(1, T, H, K, device=dev, generator=g_).bfloat16() for _ in range(3))
        g = torch.nn.functional.logsigmoid(torch.randn(1, T, H, K, device=dev, generator=g_))
        beta = torch.sigmoid(torch.randn(1, T, H, device=dev, generator=g_))
        for lst, x in ((qs, q), (ks, k), (vs, v), (gs, g), (bs, beta)):
            lst.append(x[:, :, h_lo:h_hi])
    return tuple(torch.cat(l, 0).contiguous() for l in (qs, ks, vs, gs, bs))


def run_kda(cfg, steps, warmup, dist, rank, world, peaks, lean=False):
    """The B x H (batch, head) pairs are sharded over the ranks (one global problem, strong scaling); rank 0 also runs
    all of them alone for T(1) when there is more than one rank."""
    from daisy_b200 import ops
    from daisy_b200 import accounting as acct
    B, T, H, K = cfg["B"], cfg["T"], cfg["H"], cfg["K"]
    dev = torch.device("cuda", torch.cuda.current_device())
    b_lo, b_hi, h_lo, h_hi = unit_shard(B, H, world, rank)
    q, k, v, g, beta = kda_inputs(cfg, b_lo, b_hi, h_lo, h_hi, dev)
    Bs, Hs = b_hi - b_lo, h_hi - h_lo
    res = {}

    def step():
        res["o"], _ = ops.kda_chunk_fwd(q, k, v, g, beta, None, None, False, l2norm_qk=True)

    in_bytes = sum(x.numel() * x.element_size() for x in (q, k, v, g, beta))
    flush = l2_flush_buffer(dev) if (in_bytes < 2 * L2_BYTES and not lean) else None
    ms = timed_steps(step, steps, warmup, dist, flush)
    ops.check_device_status(dev)
    per = ms / steps
    th = B * T * H                                           # global token-heads
    th_rank = Bs * T * Hs
    byts = th_rank * acct.kda_bytes_per_token_head(K, K)
    gbs = byts / (per * 1e-3) / 1e9
    if lean:
        return {"name": "kda", "ms_per_step": per, "value": th / (per * 1e-3), "unit": "token-heads/s", "steps": steps,
                "launches_per_step": 2, "roofline": None, "e2e": None,
                "config": {"workload": f"kda: B={B} T={T} H={H} K=V={K} (profiler capture case)"}}
    # e2e: host tensors in, output back
    hq, hk, hv, hg, hb = (x.cpu().pin_memory() for x in (q, k, v, g, beta))
    ho = torch.empty(res["o"].shape, dtype=res["o"].dtype).pin_memory()

    def e2e_step():
        for d_, h_ in ((q, hq), (k, hk), (v, hv), (g, hg), (beta, hb)):
            d_.copy_(h_, non_blocking=True)
        step()
        ho.copy_(res["o"], non_blocking=True)

    e2e_ms = timed_steps(e2e_step, 3, 1, dist) / 3
    del hq, hk, hv, hg, hb, ho
    strong = strong_summary(per, per, 1)
    if dist is not None:
        o = res["o"]
        gathered = [torch.empty_like(o) for _ in range(world)]
        dist.all_gather(gathered, o)
        same = None
        if rank == 0:
            full_in = kda_inputs(cfg, 0, B, 0, H, dev)
            full = {}

            def step1():
                full["o"], _ = ops.kda_chunk_fwd(*full_in, None, None, False, l2norm_qk=True)

            t1 = timed_steps(step1, steps, warmup, None) / steps
            # fewer pairs per GPU run the state pass with its K dimension split over more warps (another summation
            # order), so a shard equals the single-GPU result to bf16 rounding, not bit for bit
            diff, mag = 0.0, float(full["o"].float().abs().max())
            for r, part in enumerate(gathered):
                bl, bh_, hl, hh = unit_shard(B, H, world, r)
                diff = max(diff, float((part.float() - full["o"][bl:bh_, :, hl:hh].float()).abs().max()))
            same = bool(diff <= mag * 2.0 ** -7)
            strong = strong_summary(t1, per, world, limiter="the state pass is a serial chain over the sequence's chunks (1.5-1.9 us per "
                                                            "chunk whatever the number of (batch, head) pairs per GPU); only the intra-chunk kernel scales")
            strong["gathered_max_abs_diff"] = diff
            del full_in, full
        strong["gathered_equals_single_gpu_result"] = same
        del gathered
    kt = NCU_TRAFFIC.get("kda_per_token_head")
    return {"name": "kda_c5", "ms_per_step": per, "value": th / (per * 1e-3), "unit": "token-heads/s",
            "hbm_gbs": world * gbs, "tflops": th * acct.kda_flops_per_token_head(K, K) / (per * 1e-3) / 1e12,
            "scaling": "strong", "strong": strong,
            "steps": steps, "launches_per_step": 2, "finite": bool(torch.isfinite(res["o"].float()).all()),
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": (kt["bytes"] * th_rank) if kt else None,
                         "traffic_unit": "bytes per call, both kernels (ncu dram read+write on a reduced case, scaled by token-heads; transcribed, see traffic_source)",
                         "traffic_source": kt, "per_rank_batch_heads": Bs * Hs,
                         "kernel": "kda_intra_kernel + kda_state_kernel (one call)",
                         "peak_source": peaks["which"] + " (copy bandwidth)"},
            "e2e": {"value": th / (e2e_ms * 1e-3), "unit": "token-heads/s",
                    "h2d_bytes_per_step": th_rank * (3 * K * 2 + K * 4 + 4), "d2h_bytes_per_step": th_rank * K * 2},
            "config": {"workload": f"kda_c5: global B={B} T={T} H={H} K=V={K} chunk=64, L2-normalised q,k, "
                                   "g=logsigmoid(N(0,1)), beta=sigmoid(N(0,1)), bf16 I/O, fp32 state",
                       "per_gpu_batch_heads": Bs * Hs, "per_gpu_shape": f"B={Bs} H={Hs}",
                       "parallelism": f"(batch, head) pairs sharded {B * H} -> {Bs * Hs} per GPU over {world} GPU(s), no collective",
                       "l2": ("inputs exceed L2" if flush is None else "L2 flushed between steps (256 MiB rewrite outside the events)")}}


def run_kda_layer(cfg, steps, warmup, peaks, lean=False):
    """The row-wise passes of the KDA layer at the KDA configuration's shape (C = H*K channels), each against the
    copy bandwidth, and the whole layer's forward (dim = H*K) with its share spent in the KDA kernels."""
    from daisy_b200 import ops, B200KimiLinearSelfAttention
    B, T, H, K = cfg["B"], cfg["T"], cfg["H"], cfg["K"]
    C = H * K
    dev = torch.device("cuda", torch.cuda.current_device())
    g_ = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(B, T, C, device=dev, generator=g_).bfloat16()
    w = (torch.randn(C, 4, device=dev, generator=g_) * 0.5).bfloat16()
    o = torch.randn(B, T, H, K, device=dev, generator=g_).bfloat16()
    gate = torch.randn(B, T, H, K, device=dev, generator=g_).bfloat16()
    nw = torch.ones(K, device=dev).bfloat16()
    out = {}
    ms = timed_steps(lambda: ops.kda_short_conv(x, w), steps, warmup, None) / steps
    gbs = 2 * x.numel() * 2 / (ms * 1e-3) / 1e9
    out["short_conv"] = {"ms": ms, "hbm_gbs": gbs, "frac_of_copy": gbs / peaks["hbm_gbs"], "bytes": "read x + write y"}
    ms = timed_steps(lambda: ops.kda_out_norm(o, gate, nw), steps, warmup, None) / steps
    gbs = 3 * o.numel() * 2 / (ms * 1e-3) / 1e9
    out["out_norm"] = {"ms": ms, "hbm_gbs": gbs, "frac_of_copy": gbs / peaks["hbm_gbs"], "bytes": "read o, gate + write y"}
    a_log = torch.log(torch.empty(H, device=dev).uniform_(1, 16))
    dt_bias = torch.zeros(C, device=dev)
    ms = timed_steps(lambda: ops.kda_gate(x, a_log, K, dt_bias), steps, warmup, None) / steps
    gbs = x.numel() * 6 / (ms * 1e-3) / 1e9
    out["gate"] = {"ms": ms, "hbm_gbs": gbs, "frac_of_copy": gbs / peaks["hbm_gbs"], "bytes": "read g (bf16) + write fp32"}
    if lean:
        return {"name": "kda_layer", "ms_per_step": out["short_conv"]["ms"] + out["out_norm"]["ms"],
                "value": out["short_conv"]["hbm_gbs"], "unit": "GB/s (short_conv)", "steps": steps, "launches_per_step": 2,
                "roofline": None, "e2e": None, "passes": out,
                "config": {"workload": f"kda layer passes: B={B} T={T} C={C} (profiler capture case)"}}
    del o, gate, w
    layer = B200KimiLinearSelfAttention(C, H, T, K).to(dev).eval()
    with torch.inference_mode():
        ms = timed_steps(lambda: layer(x, None, None), max(3, steps // 2), 2, None) / max(3, steps // 2)
    out["layer_forward_ms"] = ms
    with torch.inference_mode():                                     # decode: prompt of 256 tokens, then single-token steps
        layer.reset_history()
        layer.prefill(x[:1, :256], None, None)
        x1 = x[:1, 256:257].contiguous()
        out["layer_step_us_batch1"] = timed_steps(lambda: layer.step(x1, None, None, 0, None, None, None), 50, 5, None) / 50 * 1e3
        layer.capture_step(batch=1)
        out["layer_step_graph_us_batch1"] = timed_steps(lambda: layer.step_graph(x1), 50, 5, None) / 50 * 1e3
    out["config"] = {"workload": f"kda layer: B={B} T={T} dim={C} H={H} K=V={K}, conv taps 4"}
    return out


def run_library_context(steps, warmup):
    """Context numbers, not a bench arm (``--library-context``): the GPU library calls the reference makes for the
    same work, written out here with torch / third-party calls because the reference's modules cannot travel to the
    GPU box.  (1) Its inference attention path (models/daisy/attention.py:116-127,141-154): RMS norm and rotation
    in eager torch, then ``scaled_dot_product_attention`` with the dense additive window mask, scale 0.12, at the
    headline prefill shape.  (2) The fla Triton kernels its KDA layer calls (``chunk_kda``, ``ShortConvolution``,
    ``rms_norm_gated``) at the KDA shape.  Each entry is None with a reason if the call cannot run here."""
    import torch.nn.functional as F
    from daisy_b200 import accounting
    accounting_prefill_flops = lambda: accounting.prefill_flops(*(PREFILL_C2[k] for k in ("B", "T", "H", "D", "window")))
    out = {}
    dev = torch.device("cuda", torch.cuda.current_device())
    g_ = torch.Generator(device=dev).manual_seed(3)
    B, T, H, D, W = (PREFILL_C2[k] for k in ("B", "T", "H", "D", "window"))
    try:
        q, k, v = (torch.randn(B, T, H, D, device=dev, generator=g_).bfloat16() for _ in range(3))
        ang = torch.arange(T, device=dev)[:, None] * (ROPE_BASE ** (-torch.arange(0, D, 2, device=dev) / D))[None, :]
        cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
        i = torch.arange(T, device=dev)
        allowed = (i[:, None] >= i[None, :]) & (i[:, None] - i[None, :] < W)
        mask = torch.zeros(T, T, device=dev, dtype=torch.bfloat16).masked_fill_(~allowed, float("-inf"))[None, None]

        def rope(x):
            x1, x2 = x[..., :D // 2].float(), x[..., D // 2:].float()
            return torch.cat([x1 * cos + x2 * sin, x2 * cos - x1 * sin], -1).to(x.dtype)

        def step():
            qn, kn, vn = (F.rms_norm(t, (D,)) for t in (q, k, v))
            qn, kn = rope(qn), rope(kn)
            return F.scaled_dot_product_attention(qn.transpose(1, 2), kn.transpose(1, 2), vn.transpose(1, 2),
                                                  is_causal=False, attn_mask=mask, scale=0.12)

        ms = timed_steps(step, max(2, steps // 4), 2, None) / max(2, steps // 4)
        ms_attn = timed_steps(lambda: F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                                     is_causal=False, attn_mask=mask, scale=0.12),
                              max(2, steps // 4), 1, None) / max(2, steps // 4)
        out["torch_sdpa_dense_mask"] = {"step_ms": ms, "sdpa_only_ms": ms_attn,
                                        "tflops_window_algorithmic": accounting_prefill_flops() / (ms * 1e-3) / 1e12}
        del q, k, v, mask, cos, sin
    except Exception as e:                                           # noqa: BLE001 - a context number only
        out["torch_sdpa_dense_mask"] = None
        out["torch_sdpa_reason"] = f"{type(e).__name__}: {e}"[:200]
    torch.cuda.empty_cache()
    try:
        from fla.ops.kda import chunk_kda as fla_chunk_kda
        from fla.modules import ShortConvolution
        from fla.modules.fused_norm_gate import rms_norm_gated
        B, T, H, K = (KDA_C5[k] for k in ("B", "T", "H", "K"))
        q, k, v = (torch.randn(B, T, H, K, device=dev, generator=g_).bfloat16() for _ in range(3))
        g = F.logsigmoid(torch.randn(B, T, H, K, device=dev, generator=g_))
        beta = torch.sigmoid(torch.randn(B, T, H, device=dev, generator=g_))
        with torch.no_grad():
            ms = timed_steps(lambda: fla_chunk_kda(q=q, k=k, v=v, g=g, beta=beta, use_qk_l2norm_in_kernel=True),
                             steps, warmup, None) / steps
            out["fla_chunk_kda_ms"] = ms
            conv = ShortConvolution(H * K, 4, activation="silu", dtype=torch.bfloat16).to(dev)
            x = q.view(B, T, H * K)
            out["fla_short_conv_ms"] = timed_steps(lambda: conv(x=x), steps, warmup, None) / steps
            w = torch.ones(K, device=dev, dtype=torch.bfloat16)
            out["fla_rms_norm_gated_x_sigmoid_ms"] = timed_steps(lambda: rms_norm_gated(q, k, w, None) * torch.sigmoid(k),
                                                                 steps, warmup, None) / steps
    except Exception as e:                                           # noqa: BLE001
        out["fla_reason"] = f"{type(e).__name__}: {e}"[:200]
    return out


# ----------------------------------------------------------------------------- CPU baseline / reference arm

def cpu_prefill_sample(cfg, threads=None):
    """The fp32 oracle on ONE batch row (all heads) of the prefill workload."""
    from oracle import swa
    if threads:
        torch.set_num_threads(threads)
    T, H, D, W = cfg["T"], cfg["H"], cfg["D"], cfg["window"]
    Tcap = min(T, 8192)
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(1, Tcap, H, D, generator=g).bfloat16().float() for _ in range(3))
    cos, sin = swa.rope_tables(D, Tcap, base=ROPE_BASE, truncate=False)
    t0 = time.perf_counter()
    y, _, _ = swa.swa_prefill(q, k, v, cos, sin, W, block=256)
    dt = time.perf_counter() - t0
    fl = swa.prefill_flops(1, Tcap, H, D, W)
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 of {cfg['B']} batch rows, T={Tcap}, all {H} heads, fp32 oracle, {dt:.1f} s"}, dt, fl


def host_threads() -> int:
    """Every core this process may run on.  torchrun exports OMP_NUM_THREADS=1 to its workers, which would make the
    CPU arm a single-thread run: the CPU legs set the thread count themselves."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def run_reference(args, world, rank):
    if rank != 0:
        return
    cfg = PREFILL_C2
    threads = host_threads()
    vals, fl = [], None
    for _ in range(args.warmup if args.warmup < 2 else 1):
        cpu_prefill_sample(cfg, threads)
    n = max(1, min(args.steps, 3))
    for _ in range(n):
        cb, dt, fl = cpu_prefill_sample(cfg, threads)
        vals.append(dt)
    dt = sum(vals) / len(vals)
    val = fl / dt / 1e12
    cb["value"] = val
    line = {"impl": "reference", "metric": "windowed prefill TFLOP/s", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": n, "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": f"prefill_c2: B={cfg['B']} T={cfg['T']} H={cfg['H']} D={cfg['D']} window={cfg['window']}"
                                   " (each step = bounded sample: one batch row)"},
            "cpu_baseline": cb,
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--library-context", action="store_true",
                    help="also time the GPU library calls the reference makes for the same work (context, minutes)")
    ap.add_argument("--workload", default="all", choices=["all", "prefill_c2", "prefill_c4", "prefill_bwd", "decode_c3", "kda_c5", "prefill_small", "bwd_small", "decode_small", "kda_small", "gemm_small", "kda_layer_small"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the measurements beside the workloads (projection GEMMs, generator-step latency, KDA layer "
                         "passes, the sustained loop): launch-list captures")
    args = ap.parse_args()
    world, rank, local = dist_env()
    if args.impl == "reference":
        run_reference(args, world, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: daisy_b200 has no CPU path (use --impl reference for the CPU oracle)")
    warm = max(3, args.warmup)
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    peaks = measured_peaks()
    res, extra = None, {}
    want = args.workload
    if want in ("all", "prefill_c2"):
        res = run_prefill(PREFILL_C2, args.steps, warm, dist, rank, world, peaks, "prefill_c2",
                          sustained=(want == "all" and not args.no_extras))
    if want == "prefill_small":
        res = run_prefill(PREFILL_SMALL, args.steps, args.warmup, dist, rank, world, peaks, "prefill_small", lean=True)
    if want == "bwd_small":                                  # the backward on the reduced case (profiler captures)
        res = run_prefill_bwd(PREFILL_SMALL, args.steps, args.warmup, peaks)
        res.update({"name": "prefill_bwd", "roofline": None, "e2e": None, "clocks": None})
    if want == "gemm_small":
        res = run_projection(1, 8192, 16, 128, args.steps, args.warmup, lean=True)
    if want == "decode_small":
        res = run_decode(DECODE_SMALL, args.warmup, dist, rank, world, peaks, lean=True)
    if want == "kda_small":
        res = run_kda(KDA_SMALL, args.steps, args.warmup, dist, rank, world, peaks, lean=True)
    if want == "kda_layer_small":
        res = run_kda_layer(dict(KDA_SMALL, B=4), args.steps, args.warmup, peaks, lean=True)
    if want in ("all", "prefill_c4"):
        torch.cuda.empty_cache()
        # a step shrinks with the number of ranks (heads are sharded): time as many more of them, so that the timed
        # region stays several milliseconds long
        c4 = run_prefill(PREFILL_C4, max(3, args.steps // 4) * world, warm, dist, rank, world, peaks, "prefill_c4", shard_heads=True)
        if res is None:
            res = c4
        else:
            extra["prefill_c4"] = c4
    if want in ("all", "prefill_bwd") and rank == 0 and not (want == "all" and args.no_extras):
        torch.cuda.empty_cache()
        bw = run_prefill_bwd(PREFILL_C2, max(5, args.steps // 2), warm, peaks)
        if res is None:
            bw["name"] = "prefill_bwd"; bw["roofline"] = None; bw["e2e"] = None
            res = bw
        else:
            extra["prefill_bwd"] = bw
    if want == "all" and rank == 0 and not args.no_extras:
        torch.cuda.empty_cache()
        extra["projection"] = run_projection(PREFILL_C2["B"], PREFILL_C2["T"], PREFILL_C2["H"], PREFILL_C2["D"],
                                             max(5, args.steps // 2), warm)
    if want in ("all", "decode_c3"):
        torch.cuda.empty_cache()
        d = run_decode(DECODE_C3, warm, dist, rank, world, peaks, extras=not args.no_extras)
        if res is None:
            res = d
        else:
            extra["decode"] = d
    if want in ("all", "kda_c5"):
        torch.cuda.empty_cache()
        kd = run_kda(KDA_C5, args.steps, warm, dist, rank, world, peaks)
        if res is None:
            res = kd
        else:
            extra["kda"] = kd
        if want == "all" and rank == 0 and not args.no_extras:
            torch.cuda.empty_cache()
            extra["kda_layer"] = run_kda_layer(KDA_C5, args.steps, warm, peaks)
        if args.library_context and rank == 0:
            torch.cuda.empty_cache()
            extra["library_context"] = run_library_context(args.steps, warm)
    if rank == 0:
        is_prefill = res["name"].startswith("prefill")
        nsteps = res.get("steps", args.steps)
        line = {
            "metric": "windowed prefill TFLOP/s" if is_prefill else res["name"],
            "value": res["tflops"] if is_prefill else res.get("tokens_per_s", res.get("value")),
            "unit": "TFLOP/s" if is_prefill else res.get("unit", "tokens/s"),
            "n_gpus": world, "steps": nsteps, "warmup": warm,
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": res.get("scaling", "weak"), "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": res["config"], "clocks": res.get("clocks"),
            "roofline": res["roofline"], "e2e": res["e2e"],
            "gpu_launches": res["launches_per_step"] * nsteps,
        }
        for k_ in ("strong", "sustained", "passes"):
            if k_ in res:
                line[k_] = res[k_]
        if world == 1 and not args.no_cpu_baseline and not want.endswith("_small"):
            line["cpu_baseline"] = cpu_prefill_sample(PREFILL_C2, host_threads())[0]
        else:
            line["cpu_baseline"] = None
        for k_, v_ in extra.items():
            line[k_] = {kk: vv for kk, vv in v_.items() if kk not in ("name",)}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
