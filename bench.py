#!/usr/bin/env python
"""Benchmark of the SageAttention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one full `sageattn` call (K mean, Q/K int8 quantisation, attention core) on synthetic
inputs of the named workload.  Default workload: the long-context case the headline target is
quoted on - B=1, H=64, N=32768, D=128, fp16, causal, pv_accum_dtype="fp16+fp32", HND - with the 64
heads sharded over the ranks (strong scaling, no data-path collective).

Prints ONE JSON line (rank 0).  `value` is effective attention TOPS, 4*B*H*N^2*D / t, over all
ranks, inputs resident in HBM; `e2e` is the same metric through the host-buffer API with the
host<->device copies inside the timed region; `roofline` describes the attention kernel (timed
with CUDA events inside the same steps); `cpu_baseline` is the CPU restatement of the algorithm
timed on a bounded sample; `ref_gpu` times the reference's own GPU kernels (its sm80 attention
kernel compiled for sm_100 and its Triton quantisers as cubins, oracle/_ref) on the same inputs
after the timed region; with more than one rank a second timed loop adds the exchange of the output,
every rank ending with all heads (`gather_ms_per_step`, `value_with_gather`, `gather_via`).

--impl reference times the reference itself, unmodified: when its kernels are present under
oracle/_ref and a GPU is there, its Triton quantisers + sm80 attention kernel with the fixed
(128, 64, 32, 64) configuration on the whole workload on one GPU; otherwise the CPU restatement
(oracle/) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "sageattention-autotune_b200"))
sys.path.insert(0, ROOT)

import torch

WORKLOADS = {
    # name: B, Hq, Hkv, N, D, dtype, causal, pv_accum, layout, seed
    "c5_32k": dict(B=1, Hq=64, Hkv=64, N=32768, D=128, dtype="float16", causal=True, pv="fp16+fp32", layout="HND", seed=4),
    "c5_16k": dict(B=1, Hq=64, Hkv=64, N=16384, D=128, dtype="float16", causal=True, pv="fp16+fp32", layout="HND", seed=4),
    "c5_64k": dict(B=1, Hq=64, Hkv=64, N=65536, D=128, dtype="float16", causal=True, pv="fp16+fp32", layout="HND", seed=4),
    "c5_1k": dict(B=1, Hq=64, Hkv=64, N=1024, D=128, dtype="float16", causal=True, pv="fp16+fp32", layout="HND", seed=4),
    "c5_128k": dict(B=1, Hq=64, Hkv=64, N=131072, D=128, dtype="float16", causal=True, pv="fp16+fp32", layout="HND", seed=4),
    "c5_4k": dict(B=1, Hq=64, Hkv=64, N=4096, D=128, dtype="float16", causal=True, pv="fp16+fp32", layout="HND", seed=4),
    "c5_8k_fp32": dict(B=1, Hq=32, Hkv=32, N=8192, D=128, dtype="float16", causal=False, pv="fp32", layout="HND", seed=4),
    "c5_32k_fp32": dict(B=1, Hq=64, Hkv=64, N=32768, D=128, dtype="float16", causal=True, pv="fp32", layout="HND", seed=4),
    "c2_sd": dict(B=16, Hq=10, Hkv=10, N=4096, D=64, dtype="float16", causal=False, pv="fp16+fp32", layout="HND", seed=1, k_bias=3.0),
    "c3_gqa": dict(B=4, Hq=32, Hkv=8, N=8192, D=128, dtype="bfloat16", causal=True, pv="fp32", layout="NHD", seed=2, k_outliers=20.0),
    "c4_dit_fp8": dict(B=1, Hq=24, Hkv=24, N=75600, D=128, dtype="bfloat16", causal=False, pv="fp8", layout="HND", seed=3, k_bias=2.0),
    "c4_dit": dict(B=1, Hq=24, Hkv=24, N=75600, D=128, dtype="bfloat16", causal=False, pv="fp32", layout="HND", seed=3, k_bias=2.0),
}


def bind_host_to_gpu(index: int):
    """Pin this process to the CPUs NVML reports as local to GPU `index` before any pinned host buffer
    is allocated, so that the buffers of the end-to-end leg land on the GPU's NUMA node (first touch)
    whichever core the launcher happened to start the process on.  Returns a description or None."""
    if os.environ.get("SAGE_B200_BENCH_BIND", "1") == "0":
        return {"cpus": None, "source": "unchanged (SAGE_B200_BENCH_BIND=0)"}
    try:
        import pynvml
        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(index)
        bus_id = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = [64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1]
        cpus = sorted(set(cpus) & os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return {"cpus": f"{cpus[0]}-{cpus[-1]} ({len(cpus)})", "source": "nvmlDeviceGetCpuAffinity"}
    except Exception as e:  # no NVML, no permission: run where we are
        return {"cpus": None, "source": f"unchanged ({type(e).__name__})"}
    return None


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def literal_flops(w, heads):
    return 4.0 * w["B"] * heads * w["N"] * w["N"] * w["D"]


def make_inputs(w, kv_lo, kv_hi, device, pin=False):
    """This rank's heads of the synthetic workload: N(0,1) values, optional per-channel K offset
    or outlier channels, seeded per kv-head so that the data does not depend on the sharding."""
    rep = w["Hq"] // w["Hkv"]
    dt = getattr(torch, w["dtype"])
    B, N, D = w["B"], w["N"], w["D"]
    hkv = kv_hi - kv_lo

    def shape(h):
        return (B, h, N, D) if w["layout"] == "HND" else (B, N, h, D)
    gen = torch.Generator(device=device).manual_seed(w["seed"] * 1000 + kv_lo)
    q = torch.randn(shape(hkv * rep), generator=gen, device=device, dtype=torch.float32).to(dt)
    k = torch.randn(shape(hkv), generator=gen, device=device, dtype=torch.float32)
    v = torch.randn(shape(hkv), generator=gen, device=device, dtype=torch.float32).to(dt)
    if w.get("k_bias"):
        bshape = (1, hkv, 1, D) if w["layout"] == "HND" else (1, 1, hkv, D)
        k = k + w["k_bias"] * torch.randn(bshape, generator=gen, device=device)
    if w.get("k_outliers"):
        for h in range(hkv):
            ch = torch.randperm(D, generator=gen, device=device)[:4]
            if w["layout"] == "HND":
                k[:, h, :, ch] *= w["k_outliers"]
            else:
                k[:, :, h, ch] *= w["k_outliers"]
    return q, k.to(dt), v


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

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
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples that arrived between the two host times (all of them when not given).
        The sampler is started before the warm-up so that nvidia-smi is already running when the timed
        region begins; only what it printed during that region counts."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for stamp, ln in self.lines:
            if t_begin is not None and not (t_begin <= stamp <= t_end + 0.03):
                continue
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(w, seconds_hint=20.0):
    """CPU restatement of quantise-then-attend (oracle/), all host threads, on a bounded sample:
    one head of the workload at its full sequence length when that stays near `seconds_hint`,
    otherwise a shorter sequence."""
    from oracle import sage_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = w["N"]
    est = 4.0 * n * n * w["D"] / 0.04e12 * (0.5 if w["causal"] else 1.0) * 2
    while est > seconds_hint * 1.5 and n > 1024:
        n //= 2
        est /= 4
    ws = dict(w, B=1, Hq=w["Hq"] // w["Hkv"], Hkv=1, N=n)
    q, k, v = make_inputs(ws, 0, 1, "cpu")
    t0 = time.perf_counter()
    O.sageattn(q, k, v, w["layout"], w["causal"], "fp32" if w["pv"] == "fp8" else w["pv"], True)
    dt = time.perf_counter() - t0
    tops = literal_flops(ws, ws["Hq"]) / dt / 1e12
    sample = f"B=1, {ws['Hq']} q-head(s) on 1 kv-head, N={n}, D={w['D']}, same dtype/causal/pv mode; {dt:.1f} s"
    return {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port", "sample": sample}


# dram__bytes_read.sum + dram__bytes_write.sum of the attention kernel in the ncu capture named in
# roofline.traffic_unit; re-measured whenever the kernel changes
NCU_TRAFFIC_4K = 179.6e6

REF_CFG = (128, 64, 32, 64)          # the reference's first candidate and fallback (sageattention/cuda_autotune.py:9-14)
REF_OPS = {"fp32": "qk_int8_sv_f16_accum_f32_attn", "fp16": "qk_int8_sv_f16_accum_f16_attn",
           "fp16+fp32": "qk_int8_sv_f16_accum_f16_attn_inst_buf"}


def reference_gpu_available(w) -> bool:
    from oracle import triton_ref
    so = os.path.join(ROOT, "oracle", "_ref", "libsage_ref_sm80.so")
    return torch.cuda.is_available() and os.path.exists(so) and triton_ref.available() and w["pv"] in REF_OPS


def reference_gpu_step(w):
    """One forward pass the way the reference's CUDA backend runs it (sageattention/cuda_attn.py:126-274):
    torch mean, its Triton per-thread quantisers, torch cast of V, its sm80 attention kernel.  Returns
    a callable step(q, k, v) and a dict the callable fills with per-section CUDA events."""
    from oracle import triton_ref
    torch.ops.load_library(os.path.join(ROOT, "oracle", "_ref", "libsage_ref_sm80.so"))
    op = getattr(torch.ops.sageattention_qattn_sm80, REF_OPS[w["pv"]])
    layout = w["layout"]
    seq = 2 if layout == "HND" else 1
    code = 1 if layout == "HND" else 0
    ev = {}

    def mark(name):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        ev.setdefault(name, []).append(e)

    def step(q, k, v):
        out = torch.empty_like(q)
        mark("t0")
        km = k.mean(dim=seq, keepdim=True)
        q8, qs, k8, ks = triton_ref.per_thread_int8(q, k, km, REF_CFG[0], REF_CFG[2], REF_CFG[1], REF_CFG[3], layout)
        v16 = v.to(torch.float16)
        mark("t1")
        op(q8, k8, v16, out, qs, ks, code, w["causal"], w["D"] ** -0.5, *REF_CFG, False)
        mark("t2")
        return out
    return step, ev


def run_reference(args, w):
    """--impl reference.  The reference has no CPU implementation of this path; its GPU kernels built
    from its own sources (oracle/_ref) are timed when they and a GPU are present, else the CPU
    restatement in oracle/ on a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    common = {"impl": "reference", "metric": "effective attention TOPS (4*B*H*N^2*D/t)", "unit": "TOPS",
              "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
              "scaling": "strong", "vs_baseline": None, "data": "synthetic"}
    cfg = {"workload": args.workload, **{k: w[k] for k in ("B", "Hq", "Hkv", "N", "D", "causal", "pv", "layout")}}
    if reference_gpu_available(w):
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dev = torch.device("cuda", torch.cuda.current_device())
        bind_host_to_gpu(dev.index)
        q, k, v = make_inputs(w, 0, w["Hkv"], dev)
        step, ev = reference_gpu_step(w)
        sampler = ClockSampler(dev.index)
        sampler.start()
        for _ in range(max(3, args.warmup)):
            step(q, k, v)
        torch.cuda.synchronize()
        ev.clear()
        t_begin = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step(q, k, v)
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop(t_begin, time.perf_counter())
        ms = e0.elapsed_time(e1) / args.steps
        front = sum(a.elapsed_time(b) for a, b in zip(ev["t0"], ev["t1"])) / args.steps
        attn = sum(a.elapsed_time(b) for a, b in zip(ev["t1"], ev["t2"])) / args.steps
        value = literal_flops(w, w["Hq"]) / (ms * 1e-3) / 1e12
        # end to end the way a user of the reference would run it from host memory: copy in, call, copy out
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        hout = torch.empty(hq.shape, dtype=hq.dtype, pin_memory=True)
        del q, k, v

        def step_host():
            dq, dk, dv = (t.to(dev, non_blocking=True) for t in (hq, hk, hv))
            hout.copy_(step(dq, dk, dv), non_blocking=True)
        step_host()
        torch.cuda.synchronize()
        n_e2e = max(2, min(args.steps, 5))
        e0.record()
        for _ in range(n_e2e):
            step_host()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / n_e2e
        line = dict(common, value=value, ms_per_step=ms, dtype="int8 QK^T + fp16 PV (reference sm80 mma.sync kernel)",
                    config=dict(cfg, note="the reference's own kernels, unmodified, compiled for sm_100 (oracle/_ref): Triton "
                                          "per-thread quantisers + sm80 attention kernel, fixed config (128, 64, 32, 64), whole "
                                          "workload on ONE GPU whatever --gpus says (the reference is single-GPU)"),
                    clocks=clocks, kernel_ms={"mean+quant+cast": front, "attn": attn},
                    cpu_baseline={"value": value, "unit": "TOPS", "cores": 0, "kind": "reference",
                                  "sample": "whole workload, on the GPU (the reference has no CPU path)"},
                    e2e={"value": literal_flops(w, w["Hq"]) / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_ms,
                         "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in (hq, hk, hv))),
                         "d2h_bytes_per_step": int(hout.numel() * hout.element_size()),
                         "api": "pinned host tensors copied in, the reference's call, result copied out to pinned memory"})
        print(json.dumps(line))
        return
    vals = []
    total = args.warmup + args.steps
    # keep the whole arm within a few minutes: each step is one bounded sample
    hint = max(2.0, min(20.0, 150.0 / max(1, total)))
    base = None
    t_all = time.perf_counter()
    for i in range(total):
        base = cpu_baseline(w, seconds_hint=hint)
        if i >= args.warmup:
            vals.append(base["value"])
    wall = time.perf_counter() - t_all
    value = statistics.mean(vals)
    base["value"] = value
    line = dict(common, value=value, ms_per_step=1e3 * wall / total, dtype="int8 QK^T + fp16 PV (fp32 CPU emulation)",
                config=dict(cfg, note="CPU restatement (oracle/) on host cores; each step is the bounded sample in cpu_baseline.sample"),
                cpu_baseline=base, e2e={"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line))


def run_attn_only(args, w):
    """The attention kernel alone, back to back, on one GPU: the measurement behind the tile table.
    SAGE_B200_KERNEL=coupled selects the candidate the table does not."""
    from sageattention import quant
    from sageattention.core import attn_fwd_quantized
    from sageattention.tile_table import select_entry
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    q, k, v = make_inputs(w, 0, w["Hkv"], dev)
    layout = w["layout"]
    entry = select_entry(w["D"], w["causal"], w["pv"], w["N"])
    cfg = entry["qk_config"]
    km = quant.mean_k(k, layout)
    q8, qs, k8, ks = quant.per_thread_int8(q, k, km, cfg[0], cfg[2], cfg[1], cfg[3], layout)
    v_scale = None
    if w["pv"] == "fp8":
        v16, v_scale = quant.quant_v_fp8(v, layout)
    else:
        v16 = quant.cast_v_fp16(v, layout)
    out = torch.empty_like(q)
    mode = "fp32" if w["pv"] == "fp8" else w["pv"]

    def run():
        attn_fwd_quantized(q8, k8, v16, out, qs, ks, layout, w["causal"], w["D"] ** -0.5, cfg, mode, False, "per_thread", v_scale)
    for _ in range(max(3, args.warmup)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    executed = literal_flops(w, w["Hq"]) * (0.5 if w["causal"] else 1.0)
    print(json.dumps({"attn_only": args.workload, "ms": ms, "executed_tflops": executed / (ms * 1e-3) / 1e12,
                      "table_entry": entry, "kernel_override": os.environ.get("SAGE_B200_KERNEL"), "steps": args.steps}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5_32k", choices=sorted(WORKLOADS))
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-gather", action="store_true", help="skip the second timed loop with the exchange of the output")
    ap.add_argument("--gather-via", choices=("peer", "nccl"), default="peer",
                    help="exchange of the output in the second timed loop: stores into the peers' buffers from the "
                         "attention epilogue, or the grouped NCCL all-gather")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's GPU kernels after the run")
    ap.add_argument("--attn-only", action="store_true",
                    help="time the attention kernel alone on pre-quantised inputs (tile-table sweeps) and print one line")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
        return
    if args.attn_only:
        run_attn_only(args, w)
        return

    import torch.distributed as dist
    import sageattention
    from sageattention import core as sa_core
    from sageattention.host import sageattn_host
    from sageattention.parallel import local_heads, sageattn_sharded
    from sageattention import _capi as sa_capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    host_binding = bind_host_to_gpu(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    (q_lo, q_hi), (kv_lo, kv_hi) = local_heads(w["Hq"], w["Hkv"], world, rank)
    heads_local = q_hi - q_lo
    q, k, v = make_inputs(w, kv_lo, kv_hi, dev)
    kw = dict(tensor_layout=w["layout"], is_causal=w["causal"], pv_accum_dtype=w["pv"], smooth_k=True)
    attn_call = sageattention.sageattn
    if w["pv"] == "fp8":     # e4m3 P.V variant: its own entry point, fp32 accumulation
        kw["pv_accum_dtype"] = "fp32"
        attn_call = sageattention.sageattn_qk_int8_pv_fp8_cuda

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    out_holder = {}

    def step():
        out_holder["o"] = attn_call(q, k, v, **kw) if heads_local > 0 else None

    warmup = max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    # ---- device-resident throughput: the public call as a user makes it (one C call per attention)
    for _ in range(warmup):
        step()
    barrier()
    t_begin = time.perf_counter()
    launches_before = sa_capi.lib().sage_b200_launch_count()
    total_ms = timed(step, args.steps, 0)
    launches = sa_capi.lib().sage_b200_launch_count() - launches_before      # this rank's, counted by the library
    clocks = sampler.stop(t_begin, time.perf_counter())
    # ---- the same steps once more, through the step-by-step path with CUDA events around every section
    # (quantisers, K mean, V cast, attention kernel): the per-kernel times the roofline is computed from
    sa_core._profile = []
    profiled_ms = timed(step, args.steps, 0)
    prof, sa_core._profile = sa_core._profile, None
    per_label = {}
    for label, s, e in prof:
        per_label.setdefault(label, []).append(s.elapsed_time(e))
    kern_ms = {lab: sum(v_) / len(v_) for lab, v_ in per_label.items()}
    ms_per_step = total_ms / args.steps
    F_lit = literal_flops(w, w["Hq"])
    F_exec_local = literal_flops(w, heads_local) * (0.5 if w["causal"] else 1.0)
    value = F_lit / (ms_per_step * 1e-3) / 1e12

    # ---- roofline of the attention kernel (this rank's launch)
    pk = peaks()
    attn_ms = kern_ms.get("attn")
    achieved = F_exec_local / (attn_ms * 1e-3) / 1e12 if attn_ms else None
    # half of the executed operations are int8 (2x the bf16 rate), half fp16: mixed peak = 4/3 * bf16
    peak_mixed = pk["bf16_sustained"] * 4.0 / 3.0
    roofline = {"bound": "tensor", "kernel": "sage_attn_fwd_kernel", "achieved": achieved, "peak": peak_mixed,
                "unit": "TFLOP/s", "frac": (achieved / peak_mixed) if achieved else None,
                # dram__bytes_read + dram__bytes_write of one ncu capture of this kernel (B=1, H=64, N=4096, D=128,
                # causal), scaled by this rank's Q/K/V/O element count: every term is linear in it
                "traffic": NCU_TRAFFIC_4K * (w["B"] * heads_local * w["N"] * w["D"]) / (64 * 4096 * 128) if w["D"] == 128 else None,
                "traffic_unit": "bytes per launch, scaled from the ncu capture of the B=1 H=64 N=4096 D=128 causal case",
                "peak_source": f"{pk['source']}: 4/3 x sustained dense bf16 ({pk['bf16_sustained']} TF/s); int8 counted at 2x bf16",
                "frac_of_int8_peak_literal": (literal_flops(w, heads_local) / (attn_ms * 1e-3) / 1e12) / (2 * pk["bf16_sustained"]) if attn_ms else None,
                "kernel_ms": kern_ms, "kernel_ms_pass": "second pass of the same steps, per-section CUDA events",
                "ms_per_step_profiled_pass": profiled_ms / args.steps}
    # quantisation front end against HBM: algorithmic bytes = 3 B per Q/K element + scales + mean, K counted once
    els_q = w["B"] * heads_local * w["N"] * w["D"]
    els_k = w["B"] * (kv_hi - kv_lo) * w["N"] * w["D"]
    qbytes = 3.0 * (els_q + els_k)
    front_ms = kern_ms.get("quant_q", 0.0) + kern_ms.get("smooth_quant_k", 0.0)
    roofline["quant"] = {"bound": "hbm", "achieved": qbytes / (front_ms * 1e-3) / 1e9 if front_ms else None,
                         "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": (qbytes / (front_ms * 1e-3) / 1e9) / pk["hbm_gbs"] if front_ms else None}

    # ---- the same step with the output exchanged (every rank ends with all heads): rows stored into every
    # rank's buffer by the attention epilogue, or NCCL all-gathers overlapped per head group (sageattn_sharded)
    gather_ms = plain_again_ms = gather_used = None
    if world > 1 and not args.no_gather:
        def step_gather():
            out_holder["g"] = sageattn_sharded(q, k, v, num_q_heads=w["Hq"], num_kv_heads=w["Hkv"], gather=True,
                                               attn_fn=attn_call, gather_via=args.gather_via, **kw)
        gather_ms = timed(step_gather, args.steps, 2) / args.steps
        # the plain step once more, right after: the two loops run minutes apart under a power cap, and the
        # difference between them is only meaningful next to the drift of the plain step itself
        plain_again_ms = timed(step, args.steps, 1) / args.steps
        from sageattention.parallel import last_gather_via
        gather_used = last_gather_via()            # "peer", or "nccl" when the peer buffers could not be had

    # ---- end to end from pinned host memory
    e2e = None
    if not args.no_e2e and heads_local > 0:
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        hout = torch.empty(hq.shape, dtype=hq.dtype, pin_memory=True)

        def step_host():
            sageattn_host(hq, hk, hv, out=hout, device=dev, attn_fn=attn_call, **kw)
        e2e_steps = max(2, min(args.steps, 5))
        e2e_ms = timed(step_host, e2e_steps, 1) / e2e_steps
        e2e = {"value": F_lit / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(sum(t.numel() * t.element_size() for t in (hq, hk, hv))),
               "d2h_bytes_per_step": int(hout.numel() * hout.element_size()),
               "api": "sageattention.host.sageattn_host (pinned host tensors in, pinned host tensor out)"}

    if world > 1:
        dist.barrier()
    if rank == 0:
        line = {"metric": "effective attention TOPS (4*B*H*N^2*D/t)", "value": value, "unit": "TOPS",
                "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "int8 QK^T + fp16 PV, fp32 softmax", "data": "synthetic",
                "config": {"workload": args.workload, **{k_: w[k_] for k_ in ("B", "Hq", "Hkv", "N", "D", "causal", "pv", "layout")},
                           "in_dtype": w["dtype"], "sharding": f"kv-heads over {world} rank(s), no collective in the timed region",
                           "l2": "inputs (1.6 GB per step at N=32k) exceed the 126 MB L2; no flush needed"},
                "executed_tops": value * (0.5 if w["causal"] else 1.0), "host_binding": host_binding,
                "clocks": clocks, "roofline": roofline, "e2e": e2e,
                "gpu_launches": int(launches) * world,
                "gpu_launches_note": "kernels of libsage_b200.so launched inside the timed region, counted by the library "
                                     "(sage_b200_launch_count) on rank 0, times the number of ranks",
                "gather_ms_per_step": gather_ms, "ms_per_step_after_gather_loop": plain_again_ms,
                "gather_overhead_ms": (gather_ms - 0.5 * (ms_per_step + plain_again_ms)) if gather_ms else None,
                "gather_via": gather_used if gather_ms else None,
                "value_with_gather": (F_lit / (gather_ms * 1e-3) / 1e12) if gather_ms else None}
        if not args.no_ref_gpu and world == 1 and reference_gpu_available(w):
            # the reference's own GPU kernels on the same inputs, after (never inside) the timed region
            rstep, ev = reference_gpu_step(w)
            for _ in range(2):
                rstep(q, k, v)
            torch.cuda.synchronize()
            ev.clear()
            n_ref = max(2, min(args.steps, 5))
            for _ in range(n_ref):
                rstep(q, k, v)
            torch.cuda.synchronize()
            line["ref_gpu"] = {"quant_ms": sum(a.elapsed_time(b) for a, b in zip(ev["t0"], ev["t1"])) / n_ref,
                               "attn_ms": sum(a.elapsed_time(b) for a, b in zip(ev["t1"], ev["t2"])) / n_ref,
                               "kind": "the reference's sm80 kernel compiled for sm_100 + its Triton quantisers as cubins "
                                       "(oracle/_ref), fixed config (128, 64, 32, 64), same inputs, after the timed region"}
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
