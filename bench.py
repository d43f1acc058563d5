#!/usr/bin/env python
"""Benchmark of the hot path: bf16 GEMM (headline) and attention forward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One JSON line on stdout (rank 0).  A step is one pass of the hot path over one
batch of synthetic input: for the headline workload one 8192^3 bf16 GEMM per
GPU (A row-major, B stored [N,K], fp32 accumulate, bf16 out).  With N GPUs the
global M is N x 8192, sharded into N row blocks with B replicated: no data-path
collective, weak scaling.  `value` is the whole-job TFLOP/s with inputs resident
in HBM: the MEDIAN of seven back-to-back timed regions of `--steps` launches each
(minimum and maximum beside it), plus one region of at least a second under
`roofline.sustained` (the GPU is power-capped in a long loop, so the two differ).
`e2e` is the same metric through the public call with HOST buffers (pinned host ->
device copies of the inputs and the device -> host copy of the result inside the
timed region; with several GPUs each rank uploads its own rows of A and 1/N of the
shared B, and the ranks exchange the B shards over NVLink).  The other measured
workloads (attention forward and backward, skinny and rectangular GEMMs) are timed
after the headline and reported under `other_workloads`.  With several GPUs the line
also carries `strong_scaling` (the benchmark configurations split over the GPUs by
`warpir_b200.sharding`: total work fixed) and `fused_allgather` (the GEMM with its
output all-gather fused into the epilogue against GEMM + NCCL).

`--impl reference` times the reference's own CPU computation of the same op on
the host cores, on a bounded sample of the same workload: torch.mm in fp32
(reference: tests/test_gemm_baseline.py:85) on a row block for the GEMM workloads,
the softmax(q k^T / sqrt(d)) v expression (reference: tests/test_modal_attention.py:92-98)
on a few batch x head slices for the attention workloads.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "bf16 GEMM & attn-fwd TFLOP/s per B200 (% dense peak), 1/2/4/8 GPUs"
NOMINAL_TFLOPS = 2250.0
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's kernel, from one ncu
# capture each (summaries and the exact commands: profiles/*.md); None where none was taken
NCU_DRAM_BYTES_PER_LAUNCH = {
    "gemm_8192": 1157.0e6,     # gemm_pair_sm100, band of 8 row-blocks, A tiles evict_last
    "gemm_skinny_m16": 138.3e6,
    "attn_noncausal_b16_h16_s4096_d128": 1059.3e6,
    "attn_causal_b4_h32_s8192_d128": 1058.8e6,
    "attn_bwd_causal_b4_h32_s8192_d128": 3970.4e6,     # both launches of the backward together
}

# --------------------------------------------------------------------------- workloads
GEMM_HEADLINE = dict(M=8192, N=8192, K=8192, std=1.0)


def workload_table():
    """name -> description of every measured workload (sizes per GPU)."""
    return {
        "gemm_8192": dict(kind="gemm", **GEMM_HEADLINE),
        "gemm_4096": dict(kind="gemm", M=4096, N=4096, K=4096, std=1.0),
        "gemm_2048": dict(kind="gemm", M=2048, N=2048, K=2048, std=1.0),
        "gemm_1024": dict(kind="gemm", M=1024, N=1024, K=1024, std=1.0),
        "gemm_16384x4096x8192": dict(kind="gemm", M=16384, N=4096, K=8192, std=0.02),
        "gemm_skinny_m16": dict(kind="gemm", M=16, N=8192, K=8192, std=0.02),
        "gemm_skinny_m64": dict(kind="gemm", M=64, N=8192, K=8192, std=0.02),
        "gemm_skinny_m128": dict(kind="gemm", M=128, N=8192, K=8192, std=0.02),
        "attn_noncausal_b16_h16_s4096_d128": dict(kind="attn", B=16, H=16, S=4096, D=128, causal=False),
        "attn_causal_b4_h32_s8192_d128": dict(kind="attn", B=4, H=32, S=8192, D=128, causal=True),
        "attn_causal_b4_h32_s8192_d64": dict(kind="attn", B=4, H=32, S=8192, D=64, causal=True),
        # backward of the two D = 128 configurations (FLOPs counted as five matrix products, 2.5 x forward)
        "attn_bwd_noncausal_b16_h16_s4096_d128": dict(kind="attn_bwd", B=16, H=16, S=4096, D=128, causal=False),
        "attn_bwd_causal_b4_h32_s8192_d128": dict(kind="attn_bwd", B=4, H=32, S=8192, D=128, causal=True),
    }


def flops_of(w) -> float:
    if w["kind"] == "gemm":
        return 2.0 * w["M"] * w["N"] * w["K"]
    f = 4.0 * w["B"] * w["H"] * w["S"] * w["S"] * w["D"]
    if w["kind"] == "attn_bwd":
        f *= 2.5
    return f / 2 if w["causal"] else f


def bytes_of(w) -> float:
    if w["kind"] == "gemm":
        return 2.0 * (w["M"] * w["K"] + w["N"] * w["K"] + w["M"] * w["N"])
    elems = w["B"] * w["H"] * w["S"] * w["D"]
    if w["kind"] == "attn_bwd":   # reads Q, K, V, O, dO (bf16) and LSE; writes dQ, dK, dV (fp32) and delta
        return 2.0 * 5 * elems + 4.0 * 3 * elems + 4.0 * 2 * w["B"] * w["H"] * w["S"]
    return 2.0 * 4 * elems + 4.0 * w["B"] * w["H"] * w["S"]


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks, power and throttle reasons for as long as it runs (every timed region
    of the run, not one of them); samples taken while the GPU idles between regions are told apart by
    their power draw."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "10"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows, reasons = [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in list(self.lines):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                rows.append((float(parts[0]), float(parts[1]), float(parts[2])))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": sorted(reasons)}
        top = max(r[2] for r in rows)
        loaded = [r for r in rows if r[2] >= 0.6 * top] or rows          # samples taken under load
        return {"sm_mhz": statistics.median(r[0] for r in loaded), "sm_mhz_min": min(r[0] for r in loaded),
                "sm_max_mhz": max(r[1] for r in rows), "power_w_median": statistics.median(r[2] for r in loaded),
                "samples": len(rows), "samples_under_load": len(loaded), "reasons": sorted(reasons)}


def pin_to_gpu_numa_node(index: int) -> None:
    """Run this process (and place the pinned host buffers it allocates) on the CPUs next to its GPU:
    with one process per GPU the host copies otherwise cross the socket interconnect."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, bits in enumerate(mask) for b in range(64) if (bits >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass   # best effort: a container without NVML or with a fixed cpuset simply stays where it is


# --------------------------------------------------------------------------- GPU arm
def make_inputs(w, device, seed):
    """Synthetic inputs of the workload's shapes and distributions, created on the device."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    if w["kind"] == "gemm":
        A = (torch.randn(w["M"], w["K"], generator=g, device=device) * w["std"]).bfloat16()
        B = (torch.randn(w["N"], w["K"], generator=g, device=device) * w["std"]).bfloat16()
        C = torch.empty(w["M"], w["N"], dtype=torch.bfloat16, device=device)
        return (A, B), (C,)
    shape = (w["B"], w["H"], w["S"], w["D"])
    Q, K, V = (torch.randn(shape, generator=g, device=device).bfloat16() for _ in range(3))
    O = torch.empty_like(Q)
    L = torch.empty(shape[:-1], dtype=torch.float32, device=device)
    if w["kind"] == "attn_bwd":
        from warpir_b200 import runtime
        runtime.launch_attention(Q, K, V, O, L, None, w["causal"])      # the forward's O and LSE are inputs
        dO = torch.randn(shape, generator=g, device=device).bfloat16()
        grads = tuple(torch.empty(shape, dtype=torch.float32, device=device) for _ in range(3))
        delta = torch.empty(shape[:-1], dtype=torch.float32, device=device)
        return (Q, K, V, O, dO, L), (*grads, delta)
    return (Q, K, V), (O, L)


def make_step(w, ins, outs):
    from warpir_b200 import runtime
    if w["kind"] == "gemm":
        A, B = ins
        return lambda: runtime.launch_gemm(A, B, outs[0], 1)
    if w["kind"] == "attn_bwd":
        Q, K, V, O, dO, L = ins
        dQ, dK, dV, delta = outs
        return lambda: runtime.launch_attention_backward(Q, K, V, O, dO, L, dQ, dK, dV, delta, None, w["causal"])
    Q, K, V = ins
    return lambda: runtime.launch_attention(Q, K, V, outs[0], outs[1], None, w["causal"])


def sync_all(dist_on):
    import torch
    torch.cuda.synchronize()
    if dist_on:
        import torch.distributed as dist
        dist.barrier()
        torch.cuda.synchronize()


def max_over_ranks(ms: float, dist_on: bool, device) -> float:
    if not dist_on:
        return ms
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(step, steps, warmup, dist_on, device):
    """W untimed steps, then exactly `steps` steps between two CUDA events on the
    launching (current) stream, bracketed by barrier + synchronize; max over ranks."""
    import torch
    for _ in range(warmup):
        step()
    sync_all(dist_on)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    sync_all(dist_on)
    return max_over_ranks(e0.elapsed_time(e1), dist_on, device)


REGIONS = 7   # timed regions per measurement: the median is reported, minimum and maximum beside it


def time_regions(timer, step, steps, warmup, dist_on, device, regions=REGIONS):
    """`regions` back-to-back timed regions of `steps` launches each (warm-up before the first only)."""
    out = [timer(step, steps, warmup, dist_on, device)]
    out += [timer(step, steps, 0, dist_on, device) for _ in range(regions - 1)]
    return out


def time_regions_graph(step, steps, warmup, dist_on, device, regions=REGIONS):
    """Same contract as time_regions for steps that last only microseconds: the K launches are
    captured once into a CUDA graph and each timed region is one replay, so a region holds K kernel
    launches and no per-launch host work (a Python call costs more than such a kernel runs)."""
    import torch
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(steps):
                step()
    torch.cuda.synchronize()
    graph.replay()                      # one untimed replay
    out = []
    for _ in range(regions):
        sync_all(dist_on)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        sync_all(dist_on)
        out.append(max_over_ranks(e0.elapsed_time(e1), dist_on, device))
    return out


def time_e2e(w, steps, warmup, dist_on, device, world=1, rank=0):
    """Same step through the public call with HOST buffers: every step copies its inputs from
    pinned host memory and reads its result back into pinned host memory.  As a real caller
    would, the copies of neighbouring steps are overlapped with the kernel on two side streams
    (device buffers are double-buffered); every byte of every step is still moved inside the
    timed region, which starts and ends on the launching stream.

    Several GPUs, GEMM: B is the one operand all ranks share.  Each rank uploads its own rows of A
    and ONE N-th of B over PCIe, and the ranks exchange the B shards over NVLink (NCCL all-gather,
    inside the timed region, on the input stream) instead of every rank pulling the whole B through
    the host's memory system."""
    import torch
    sets = [make_inputs(w, device, seed=1234 + k) for k in range(2)]
    shard_b = dist_on and w["kind"] == "gemm" and w["N"] % world == 0
    h_ins = [t.cpu().pin_memory() for t in sets[0][0]]
    b_rows = None
    if shard_b:
        b_rows = w["N"] // world
        h_ins[1] = sets[0][0][1][rank * b_rows:(rank + 1) * b_rows].cpu().pin_memory()   # this rank's share of B
        b_shard_dev = [torch.empty(b_rows, w["K"], dtype=torch.bfloat16, device=device) for _ in range(2)]
    h_outs = [[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs] for _, outs in sets]
    steps_fn = [make_step(w, ins, outs) for ins, outs in sets]
    main = torch.cuda.current_stream(device)
    s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    state = {"i": 0}

    def e2e_step():
        i = state["i"]
        b = i & 1
        ins, outs = sets[b]
        s_in.wait_stream(main) if i == 0 else None
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_comp[b])          # the kernel that last read this buffer is done
            if shard_b:
                import torch.distributed as dist
                ins[0].copy_(h_ins[0], non_blocking=True)
                b_shard_dev[b].copy_(h_ins[1], non_blocking=True)
                dist.all_gather_into_tensor(ins[1], b_shard_dev[b])     # B shards cross NVLink, not PCIe
            else:
                for d, h in zip(ins, h_ins):
                    d.copy_(h, non_blocking=True)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        if i >= 2:
            main.wait_event(ev_out[b])               # the previous result of this buffer has left
        steps_fn[b]()
        ev_comp[b].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            for d, h in zip(outs, h_outs[b]):
                h.copy_(d, non_blocking=True)
            ev_out[b].record(s_out)
        state["i"] = i + 1

    def drain():
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    for _ in range(warmup):
        e2e_step()
    drain()
    sync_all(dist_on)
    state["i"] = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        e2e_step()
    drain()
    e1.record()
    sync_all(dist_on)
    ms = max_over_ranks(e0.elapsed_time(e1), dist_on, device)
    h2d = sum(t.numel() * t.element_size() for t in h_ins)
    d2h = sum(t.numel() * t.element_size() for t in h_outs[0])
    extra = {}
    if shard_b:
        extra = {"b_upload": f"each rank uploads rows {b_rows} of {w['N']} of B; NCCL all-gather of the shards inside the timed region",
                 "nvlink_bytes_per_step_per_rank": 2 * b_rows * w["K"] * (world - 1)}
    return ms, h2d, d2h, extra


def cpu_baseline_gemm(w, target_seconds=10.0):
    """The oracle (the reference's torch.mm expression on CPU, fp32) on a row-block
    sample of the workload, all host threads."""
    import torch
    from oracle import reference_ops as R
    cores = R.host_threads()
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    N, K = w["N"], w["K"]
    B = R.randn_bf16((N, K), g, w["std"])
    rows = min(256, w["M"])
    A = R.randn_bf16((rows, K), g, w["std"])
    t0 = time.perf_counter()
    R.gemm_ref(A, B, 1)
    dt = time.perf_counter() - t0
    scale = max(1, min(w["M"] // rows, int(target_seconds / max(dt, 1e-3))))
    rows2 = rows * scale
    A = R.randn_bf16((rows2, K), g, w["std"])
    t0 = time.perf_counter()
    R.gemm_ref(A, B, 1)
    dt = time.perf_counter() - t0
    return {"value": 2.0 * rows2 * N * K / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"rows 0..{rows2} of A ({rows2}x{K}) times the full B ({N}x{K}), fp32 torch.mm, {dt:.2f} s"}


def _attention_slices(w, n, seed=0):
    """Inputs of `n` batch x head slices of an attention workload (every slice costs the same)."""
    from oracle import reference_ops as R
    return R.attention_inputs(1, n, w["S"], w["D"], seed=seed)


def cpu_baseline_attn(w, target_seconds=10.0):
    """The oracle's one-head expression (softmax(q k^T / sqrt(d)) v in fp32 on CPU, the reference's
    `_ref_attention` plus the causal mask and log-sum-exp) on as many batch x head slices as fit in
    about `target_seconds`; a rate, counted with the workload's own FLOP convention."""
    import torch
    from oracle import reference_ops as R
    cores = R.host_threads()
    torch.set_num_threads(cores)
    Q, K, V = _attention_slices(w, 1)
    t0 = time.perf_counter()
    R.attention_slice_ref(Q[0, 0], K[0, 0], V[0, 0], None, w["causal"])
    dt = time.perf_counter() - t0
    n = max(1, min(w["B"] * w["H"], int(target_seconds / max(dt, 1e-3))))
    Q, K, V = _attention_slices(w, n, seed=1)
    t0 = time.perf_counter()
    for h in range(n):
        R.attention_slice_ref(Q[0, h], K[0, h], V[0, h], None, w["causal"])
    dt = time.perf_counter() - t0
    per_slice = flops_of(w) / (w["B"] * w["H"])
    return {"value": n * per_slice / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{n} of the {w['B'] * w['H']} batch x head slices (S={w['S']}, D={w['D']}, causal={w['causal']}), "
                      f"fp32 torch on CPU, {dt:.2f} s; the rate does not depend on the slice"}


# --------------------------------------------------------------------------- arms
def run_reference_arm(args, w, name):
    """The reference's CPU computation of the op on the host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    from oracle import reference_ops as R
    cores = R.host_threads()
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    if w["kind"] == "gemm":
        N, K = w["N"], w["K"]
        rows = min(w["M"], 1024)                      # bounded sample: a row block of A, the full B
        A = R.randn_bf16((rows, K), g, w["std"])
        B = R.randn_bf16((N, K), g, w["std"])
        work = 2.0 * rows * N * K
        sample = f"rows 0..{rows} of A ({rows}x{K}) times the full B ({N}x{K}) per step, fp32 torch.mm on CPU"

        def one():
            R.gemm_ref(A, B, 1)
    elif w["kind"] == "attn":
        n = 2                                         # bounded sample: two batch x head slices per step
        Q, K, V = _attention_slices(w, n)
        work = n * flops_of(w) / (w["B"] * w["H"])
        sample = (f"{n} of the {w['B'] * w['H']} batch x head slices per step (S={w['S']}, D={w['D']}, "
                  f"causal={w['causal']}), fp32 torch softmax(q k^T / sqrt(d)) v on CPU")

        def one():
            for h in range(n):
                R.attention_slice_ref(Q[0, h], K[0, h], V[0, h], None, w["causal"])
    else:
        raise SystemExit("the reference has no backward to time: the reference arm covers the GEMM and attention-forward workloads")
    for _ in range(max(1, min(args.warmup, 3))):
        one()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one()
    dt = time.perf_counter() - t0
    value = work * args.steps / dt / 1e12
    emit({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32 on CPU (bf16 inputs)", "data": "synthetic",
        "config": {"workload": name, **{k: v for k, v in w.items() if k != "kind"}, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def measure_workload(name, w, steps, warmup, dist_on, device, world, peaks, regions=3):
    ins, outs = make_inputs(w, device, seed=1000 + int(os.environ.get("RANK", "0")))
    step = make_step(w, ins, outs)
    small = flops_of(w) < 4e10          # well under 100 us per step: launch-bound from Python
    if small:
        times = time_regions_graph(step, steps, warmup, dist_on, device, regions)
    else:
        times = time_regions(time_steps, step, steps, warmup, dist_on, device, regions)
    per = statistics.median(times) / steps
    tf = flops_of(w) * world / per / 1e9
    rec = {"workload": name, "ms_per_step": per, "ms_per_step_min": min(times) / steps, "ms_per_step_max": max(times) / steps,
           "regions": regions, "steps_per_region": steps,
           "timed_as": "cuda graph of the steps" if small else "stream launches",
           "tflops": tf, "tflops_per_gpu": tf / world,
           "frac_of_nominal_2250": tf / world / NOMINAL_TFLOPS,
           "frac_of_measured_burst": tf / world / peaks["bf16_tflops"],
           "hbm_gbs_per_gpu": bytes_of(w) / per / 1e6,
           "frac_of_measured_hbm": bytes_of(w) / per / 1e6 / peaks["hbm_gbs"]}
    del ins, outs
    return rec


def shard_workload(w, world, rank):
    """This rank's part of workload `w` when the job's total work is FIXED and split over `world` GPUs
    by warpir_b200.sharding: row blocks of A and C (column blocks of B and C for skinny GEMMs), or
    contiguous batch x head slices; None when the rank's share is empty."""
    from warpir_b200 import sharding
    if w["kind"] == "gemm":
        sh = sharding.gemm_shard(w["M"], w["N"], world, rank)
        m = sh["rows"][1] - sh["rows"][0]
        n = sh["cols"][1] - sh["cols"][0]
        if m <= 0 or n <= 0:
            return None, sh["axis"]
        return dict(w, M=m, N=n), sh["axis"]
    b0, b1 = sharding.attention_shard(w["B"], w["H"], world, rank)
    if b1 <= b0:
        return None, "batch x head"
    return dict(w, B=1, H=b1 - b0), "batch x head"


def measure_strong_scaling(steps, warmup, device, world, rank, names):
    """Every benchmark configuration with its total work fixed and split over the GPUs (no data-path
    collective): time = max over ranks of the shard's time, efficiency against the same GPUs running the
    whole problem alone (measured here, on every rank, max over ranks)."""
    table = workload_table()
    out = []
    for name in names:
        w = table[name]
        small = flops_of(w) < 4e10
        k = steps if not small else max(steps, 50)
        timer = time_regions_graph if small else (lambda st, n, wu, d, dev, r: time_regions(time_steps, st, n, wu, d, dev, r))
        ins, outs = make_inputs(w, device, seed=2000 + rank)
        t_full = statistics.median(timer(make_step(w, ins, outs), k, warmup, True, device, 3)) / k
        del ins, outs
        part, axis = shard_workload(w, world, rank)
        if part is not None:
            ins, outs = make_inputs(part, device, seed=3000 + rank)
            step = make_step(part, ins, outs)
        else:
            step = lambda: None
        t_shard = statistics.median(timer(step, k, warmup, True, device, 3)) / k
        tf = flops_of(w) / t_shard / 1e9
        out.append({"workload": name, "split": axis, "shard": {a: b for a, b in (part or {}).items() if a in ("M", "N", "K", "B", "H", "S", "D")},
                    "ms_per_step": t_shard, "ms_per_step_one_gpu_whole_problem": t_full,
                    "tflops_total": tf, "tflops_per_gpu": tf / world,
                    "speedup": t_full / t_shard, "efficiency": t_full / t_shard / world})
    return out


def measure_allgather(w, steps, device, world, rank):
    """Row-sharded GEMM whose output every GPU needs whole: the fused epilogue all-gather
    (`warpir_gemm_bf16_allgather`, stores to peers over NVLink from the GEMM itself) against the
    same GEMM followed by NCCL's all-gather.  Times are device events, max over ranks."""
    import torch
    import torch.distributed as dist
    from warpir_b200 import runtime, sharding
    M, N, K = w["M"], w["N"], w["K"]
    g = torch.Generator(device=device).manual_seed(77 + rank)
    A = (torch.randn(M, K, generator=g, device=device) * w["std"]).bfloat16()
    B = (torch.randn(N, K, generator=torch.Generator(device=device).manual_seed(78), device=device) * w["std"]).bfloat16()
    out = sharding.GatheredOutput(world * M, N)
    block = torch.empty(M, N, dtype=torch.bfloat16, device=device)
    full = torch.empty(world * M, N, dtype=torch.bfloat16, device=device)

    def fused():
        sharding.gemm_allgather(A, B, out, rank * M)

    def separate():
        runtime.launch_gemm(A, B, block, 1)
        dist.all_gather_into_tensor(full, block)

    res = {}
    for tag, fn in (("gemm_plus_nccl_allgather", separate), ("fused", fused)):
        ms = time_steps(fn, steps, 3, True, device)
        res[tag + "_ms_per_step"] = ms / steps
    out.wait_all()
    # same bytes everywhere, and equal to what NCCL gathered
    same = bool(torch.equal(out.tensor.view(torch.int16), full.view(torch.int16)))
    flag = torch.tensor([1 if same else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    runtime.read_status(device)
    res.update({"matches_nccl_on_every_rank": bool(flag.item()), "rows_per_gpu": M, "N": N, "K": K,
                "bytes_sent_per_gpu": 2.0 * M * N * (world - 1), "steps": steps,
                "nvlink_gbs_per_gpu_fused": 2.0 * M * N * (world - 1) / (res["fused_ms_per_step"] * 1e6)})
    return res


def run_gpu_arm(args, w, name):
    import torch
    from warpir_b200 import runtime
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist_on = world > 1
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    pin_to_gpu_numa_node(local)
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    runtime.load_library()  # raises if the compiled library is missing
    if dist_on:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    peaks, peak_src = load_peaks()

    ins, outs = make_inputs(w, device, seed=1000 + rank)
    step = make_step(w, ins, outs)
    small = flops_of(w) < 4e10
    sampler = ClockSampler(local)
    for _ in range(args.warmup):
        step()
    sampler.start()
    # nvidia-smi needs a moment to come up: keep the GPU under the same load (extra untimed steps)
    # until its first sample is in, so that the samples cover the timed regions from the start
    t_wait = time.perf_counter()
    while sampler.proc is not None and not sampler.lines and time.perf_counter() - t_wait < 2.0:
        step()
        torch.cuda.synchronize()
    if small:
        times = time_regions_graph(step, args.steps, 0, dist_on, device, args.regions)
    else:
        times = time_regions(time_steps, step, args.steps, 0, dist_on, device, args.regions)
    ms = statistics.median(times)
    per = ms / args.steps
    value = flops_of(w) * world / per / 1e9          # TFLOP/s, whole job
    # one long region: under the power cap the clock settles well below what a 20-step burst sees
    sustained = None
    if not small and args.sustained:
        n_long = max(args.steps, int(math.ceil(1100.0 / per)))
        ms_long = time_steps(step, n_long, 0, dist_on, device)
        sustained = {"steps": n_long, "seconds": ms_long / 1e3, "ms_per_step": ms_long / n_long,
                     "tflops_per_gpu": flops_of(w) / (ms_long / n_long) / 1e9}
    clocks = sampler.stop()
    runtime.read_status(device)
    del ins, outs

    e2e = None
    if args.e2e:
        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms, h2d, d2h, extra = time_e2e(w, e2e_steps, 3, dist_on, device, world, rank)
        e2e = {"value": flops_of(w) * world / (e2e_ms / e2e_steps) / 1e9, "unit": "TFLOP/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "ms_per_step": e2e_ms / e2e_steps, "bytes_are": "per rank", **extra}

    tensor_bound = w["kind"] != "gemm" or min(w["M"], w["N"]) > 1024
    if tensor_bound:
        peak = peaks["bf16_tflops"]            # each timed region is a burst of `steps` launches
        achieved = flops_of(w) / per / 1e9
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": f"{peak_src} burst cuBLAS bf16 (a region is {ms:.0f} ms)",
                "frac_of_nominal_2250": achieved / NOMINAL_TFLOPS, "traffic": None,
                # the regions straddle the onset of the power cap (tens of milliseconds into the load): the
                # fastest region is the figure to hold against a best-of-N burst peak
                "best_region": {"achieved": flops_of(w) / (min(times) / args.steps) / 1e9,
                                "frac": flops_of(w) / (min(times) / args.steps) / 1e9 / peak}}
        if sustained is not None:
            roof["sustained"] = {"achieved": sustained["tflops_per_gpu"], "peak": peaks["bf16_tflops_sustained"],
                                 "frac": sustained["tflops_per_gpu"] / peaks["bf16_tflops_sustained"],
                                 "peak_source": f"{peak_src} sustained cuBLAS bf16", "seconds": sustained["seconds"],
                                 "steps": sustained["steps"],
                                 "frac_of_nominal_2250": sustained["tflops_per_gpu"] / NOMINAL_TFLOPS}
    else:
        achieved = bytes_of(w) / per / 1e6
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_src} copy bandwidth", "traffic": None}
    roof["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH.get(name)
    roof["traffic_unit"] = "bytes per launch (ncu dram read + write)"
    roof["algorithmic_bytes_per_launch"] = bytes_of(w)
    roof["kernel"] = {"gemm": "gemm_pair_sm100" if (w["kind"] == "gemm" and min(w["M"], w["N"]) >= 2048) else "gemm_bf16_sm100",
                      "attn": "attn_fwd_sm100" if (w.get("causal") and w.get("D") == 128) else "attn_fwd_wide_sm100",
                      "attn_bwd": "attn_bwd_wide_sm100"}[w["kind"]]
    roof["algorithmic_per_launch"] = flops_of(w) if tensor_bound else bytes_of(w)

    others = []
    if args.others:
        table = workload_table()
        for oname, ow in table.items():
            if oname == name:
                continue
            k = 10 if flops_of(ow) > 5e10 else 50     # three regions of k launches each
            # Each workload starts from a GPU that has idled for half a second, as a run of it alone would, and
            # carries the clock it ran at (when its regions are long enough for the sampler to see): timed right
            # behind the headline's seconds at the power cap, the same kernels measured up to 25 % slower than alone.
            time.sleep(0.5)
            osampler = ClockSampler(local)
            osampler.start()
            rec = measure_workload(oname, ow, k, 5, dist_on, device, world, peaks)
            oc = osampler.stop()
            rec["sm_mhz"] = oc.get("sm_mhz")
            rec["clock_reasons"] = oc.get("reasons")
            others.append(rec)
        runtime.read_status(device)

    strong = None
    if dist_on and args.strong:
        strong = measure_strong_scaling(10, 3, device, world, rank,
                                        ["gemm_8192", "gemm_4096", "gemm_skinny_m16", "gemm_skinny_m64", "gemm_skinny_m128",
                                         "attn_noncausal_b16_h16_s4096_d128", "attn_causal_b4_h32_s8192_d128",
                                         "attn_causal_b4_h32_s8192_d64"])
        runtime.read_status(device)

    gathered = None
    if args.allgather and dist_on:
        gathered = measure_allgather(workload_table()["gemm_8192"], 20, device, world, rank)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline_gemm(w) if w["kind"] == "gemm" else \
            cpu_baseline_attn(w if w["kind"] == "attn" else dict(w, kind="attn"))

    if dist_on:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    if clocks.get("sm_mhz"):
        clocks["ms_per_step_x_ghz"] = per * clocks["sm_mhz"] / 1e3    # time at 1 GHz: compares runs at different clocks
    line = {
        "metric": METRIC,
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": name, **{k: v for k, v in w.items() if k != "kind"},
                   "per_gpu": "sizes above are per GPU; the job is n_gpus such shards",
                   "sharding": f"{world} independent row blocks of M (B replicated), no collective"
                   if w["kind"] == "gemm" else f"batch x head slices split over {world} GPUs, no collective",
                   "l2": "inputs+outputs per step exceed the 126 MB L2" if bytes_of(w) > 126e6
                   else "working set fits in L2 (not flushed)"},
        "timed_regions": {"count": len(times), "steps_per_region": args.steps, "value_is": "median",
                          "tflops_min": flops_of(w) * world / (max(times) / args.steps) / 1e9,
                          "tflops_max": flops_of(w) * world / (min(times) / args.steps) / 1e9,
                          "ms_per_region": times},
        "sustained": sustained,
        "clocks": clocks, "gpu_launches": args.steps,
        "e2e": e2e,
        "roofline": roof,
        "cpu_baseline": cpu,
        "frac_of_nominal_2250_per_gpu": value / world / NOMINAL_TFLOPS,
        "other_workloads": others,
    }
    if strong is not None:
        line["strong_scaling"] = strong
    if gathered is not None:
        line["fused_allgather"] = gathered
    emit(line)


_JSON_FD = None


def reserve_stdout():
    """Keeps stdout for the one JSON line: everything else that writes to file descriptor 1
    from here on (NCCL announces its version there, whatever NCCL_DEBUG says) goes to stderr."""
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="warpir_b200", choices=["warpir_b200", "reference"])
    ap.add_argument("--workload", default="gemm_8192", choices=sorted(workload_table()))
    ap.add_argument("--no-others", dest="others", action="store_false", help="skip the secondary workloads")
    ap.add_argument("--no-e2e", dest="e2e", action="store_false", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-allgather", dest="allgather", action="store_false",
                    help="with --gpus > 1: skip the GEMM with its output all-gather fused into the epilogue")
    ap.add_argument("--allgather", dest="allgather", action="store_true", help=argparse.SUPPRESS)   # the default
    ap.add_argument("--regions", type=int, default=REGIONS, help="timed regions of --steps launches each (median reported)")
    ap.add_argument("--no-sustained", dest="sustained", action="store_false",
                    help="skip the region of at least a second (for profiler captures, which want few launches)")
    ap.add_argument("--no-strong", dest="strong", action="store_false",
                    help="with --gpus > 1: skip the strong-scaling runs (fixed total work split over the GPUs)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl != "reference":
        args.warmup = 3
    w = workload_table()[args.workload]
    reserve_stdout()
    if args.impl == "reference":
        run_reference_arm(args, w, args.workload)
    else:
        run_gpu_arm(args, w, args.workload)


if __name__ == "__main__":
    main()
