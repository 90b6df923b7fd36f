#!/usr/bin/env python
"""Benchmark of the sequence-parallel cross-attention layer (forward + backward), one JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 2]

Workload (N = 1..8, total work fixed => strong scaling): B=1, Hq=32, Hkv=8, D=128, Sq=2048 text queries,
Skv=131072 visual keys, bf16, no mask, scale 1/sqrt(128); Q/dO and K/V are sharded evenly by sequence over
the N ranks (rank r takes the r-th slice, reference test.py:164-178). Inputs are seeded synthetic tensors
(q,k,v ~ N(0,0.5^2), dO ~ N(0,1), reference test.py:101-107).

A step = one forward + one backward of the layer through lv_xattn_b200._attn_forward/_attn_backward.
  value   whole-job algorithmic TFLOP/s (3.5 * 4*Hq*D*Sq*Skv per step over all ranks), inputs resident in HBM,
          device time from CUDA events summed over the K steps, max over ranks
  e2e     the same through lv_xattn_b200.HostStreamedAttention.step with HOST (pinned) inputs and outputs:
          H2D of q,k,v,dO and D2H of o,dq,dk,dv inside the timed region (at N=1 the K/V shard is streamed in
          chunks so that the kernels overlap the copies)
  roofline  the backward block kernel: algorithmic FLOPs of its launches / its event-timed duration, against
          the measured bf16 tensor peak
  cpu_baseline  the CPU oracle (reference test.py:129-156 math) timed on the host cores on a bounded sample
--impl reference times that CPU path alone (the reference's GPU path is Triton and is not part of this build).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

CONFIGS = {
    # id: (B, Hq, Hkv, D, Sq, Skv, dtype)
    1: (1, 32, 8, 128, 512, 8192, "bf16"),
    2: (1, 32, 8, 128, 2048, 131072, "bf16"),
}
METRIC = "xattn_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": p.get("bf16_tflops"), "bf16_sustained": p.get("bf16_tflops_sustained"),
                "hbm_gbs": p.get("hbm_gbs"), "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[1]))
                mx = max(mx, float(s[2]))
                for n, v in zip(names, s[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        sm.sort()
        # samples taken under load: the upper half of the distribution (idle samples sit at the floor)
        load = sm[len(sm) // 2:] if sm else []
        med = load[len(load) // 2] if load else None
        return {"sm_mhz": med, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def gen_inputs(cfg, rank, world, seed, device, dtype):
    """Seeded full-tensor statistics, generated shard-wise on the device (each rank only its slices)."""
    B, Hq, Hkv, D, Sq, Skv, _ = cfg
    g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    Sl, Kl = Sq // world, Skv // world
    q = torch.empty(B, Hq, Sl, D, device=device).normal_(0, 0.5, generator=g).to(dtype)
    k = torch.empty(B, Hkv, Kl, D, device=device).normal_(0, 0.5, generator=g).to(dtype)
    v = torch.empty(B, Hkv, Kl, D, device=device).normal_(0, 0.5, generator=g).to(dtype)
    do = torch.empty(B, Hq, Sl, D, device=device).normal_(0, 1.0, generator=g).to(dtype)
    return q, k, v, do


def cpu_attention_sample(cfg, threads, heads):
    """The CPU oracle on a bounded sample of the workload: `heads` query heads (one KV group at a time, one
    head per pass so that a [Sq, Skv] fp32 score matrix stays near 1 GiB), all Sq queries, all Skv keys.
    Returns (TFLOP/s, seconds, description)."""
    from oracle import attention_oracle as orc
    B, Hq, Hkv, D, Sq, Skv, _ = cfg
    torch.set_num_threads(threads)
    q, k, v, do = orc.make_inputs(B, heads, 1, Sq, Skv, D, 1, torch.float32)
    t0 = time.perf_counter()
    for h in range(heads):
        orc.attention_fwd_bwd(q[:, h:h + 1], k, v, do[:, h:h + 1], 1.0 / math.sqrt(D))
    dt = time.perf_counter() - t0
    f_fwd, f_bwd = orc.flops_fwd_bwd(B, heads, D, Sq, Skv)
    desc = (f"fp32 torch CPU fwd+bwd (reference test.py:129-156 math), {heads} of {Hq} query heads, "
            f"Sq={Sq} Skv={Skv} ({heads}/{Hq} of the workload's FLOPs)")
    return (f_fwd + f_bwd) / dt / 1e12, dt, desc


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals = []
    for i in range(args.warmup + args.steps):
        tf, dt, desc = cpu_attention_sample(cfg, threads, 4)
        if i >= args.warmup:
            vals.append((tf, dt))
    tf = sum(v[0] for v in vals) / len(vals)
    ms = 1e3 * sum(v[1] for v in vals) / len(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.config, cfg), "note": "each step is the bounded CPU sample"},
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_name(cid, cfg):
    B, Hq, Hkv, D, Sq, Skv, dt = cfg
    return f"config{cid}: xattn fwd+bwd B={B} Hq={Hq} Hkv={Hkv} D={D} Sq={Sq} Skv={Skv} {dt}, Q and K/V sharded by sequence"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="K/V chunks of the host-streamed end-to-end step")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    if args.impl == "reference":
        run_reference(args, cfg)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the library has no CPU path)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    import lv_xattn_b200 as lvx
    from lv_xattn_b200 import ops, _lib
    from oracle import attention_oracle as orc  # FLOP formula only

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if "LVX_NCCL_DEBUG" in os.environ:
            os.environ["NCCL_DEBUG"] = os.environ["LVX_NCCL_DEBUG"]
        else:
            os.environ.pop("NCCL_DEBUG", None)      # any level prints NCCL's version banner on stdout
        lvx.initialize_distributed("nccl")

    B, Hq, Hkv, D, Sq, Skv, dts = cfg
    dtype = torch.bfloat16
    scale = 1.0 / math.sqrt(D)
    q, k, v, do = gen_inputs(cfg, rank, world, 1, dev, dtype)
    f_fwd, f_bwd = orc.flops_fwd_bwd(B, Hq, D, Sq, Skv)
    flops_step = f_fwd + f_bwd
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB L2

    def step_device():
        _, _, _, o, L = lvx._attn_forward(q, k, v, False, scale, None)
        return lvx._attn_backward(do, q, k, v, o, L, False, scale, None, "flash") + (o,)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        evs = []
        wall0 = time.perf_counter()
        for _ in range(steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            evs.append((a, b))
        barrier()
        wall = (time.perf_counter() - wall0) * 1e3
        ms = sum(a.elapsed_time(b) for a, b in evs)
        t = torch.tensor([ms, wall], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t[0].item(), t[1].item()

    # ---- device-resident run (value + roofline of the dominant kernel) -----------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()                      # nvidia-smi needs a moment before its first sample
    for _ in range(args.warmup):
        step_device()
    barrier()
    ops.set_profiling(True)
    ops.launch_count = 0
    n_before = len(sampler.samples)
    total_ms, wall_ms = timed(step_device, args.steps, 0)
    sampler.samples = sampler.samples[n_before:] or sampler.samples[-1:]
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.launch_count
    prof = ops.take_profile()
    ops.set_profiling(False)
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"device status word {status:#x}: a bounded wait ran out")
    ms_per_step = total_ms / args.steps
    value = flops_step / (ms_per_step * 1e-3) / 1e12

    pk = peaks()
    # dominant kernel: the backward block. Its launches of one step together do f_bwd/world FLOPs on this rank.
    bwd_ms_step = sum(prof["bwd"]) / args.steps
    fwd_ms_step = sum(prof["fwd"]) / args.steps
    achieved = (f_bwd / world) / (bwd_ms_step * 1e-3) / 1e12
    peak = pk["bf16_sustained"]
    roofline = {"bound": "tensor", "kernel": "bwd_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "peak_source": f"{pk['source']} (sustained cuBLAS bf16)",
                # DRAM bytes per launch, from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum) of one
                # launch at Sq=2048, Skv=32768: 324.5 MB, of which 268.4 MB is K,V in and dK,dV out (scales with
                # this rank's key rows) and 56 MB is Q, dO and dQ (all query blocks pass through every rank)
                "traffic": 268.4e6 * (Skv / world) / 32768 + 56e6 * (Sq / 2048),
                "traffic_source": "ncu capture at Skv=32768 scaled by key rows",
                "bwd_kernel_ms_per_step": bwd_ms_step, "fwd_kernel_ms_per_step": fwd_ms_step,
                "fwd_achieved": (f_fwd / world) / (fwd_ms_step * 1e-3) / 1e12,
                "launches_per_step": {"fwd": len(prof["fwd"]) // args.steps, "bwd": len(prof["bwd"]) // args.steps}}

    # ---- end-to-end run: host (pinned) inputs, results read back ------------------------------------
    e2e = None
    if not args.no_e2e:
        hq, hk, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, do))
        ho, hdq = torch.empty_like(hq).pin_memory(), torch.empty_like(hq).pin_memory()
        hdk, hdv = torch.empty_like(hk).pin_memory(), torch.empty_like(hv).pin_memory()

        streamer = lvx.HostStreamedAttention(dev, chunks=args.e2e_chunks)

        def step_e2e():
            streamer.step(hq, hk, hv, hdo, scale, ho, hdq, hdk, hdv)

        e_steps = max(1, min(args.steps, 5))
        e_ms, _ = timed(step_e2e, e_steps, 1)
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
        d2h = sum(t.numel() * t.element_size() for t in (ho, hdq, hdk, hdv))
        e2e = {"value": flops_step / (e_ms / e_steps * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e_ms / e_steps,
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e_steps}

    # ---- CPU baseline (rank 0, N=1 only) ----------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tf, dt, desc = cpu_attention_sample(cfg, threads, 16)
        cpu = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc, "seconds": dt}

    if rank == 0:
        roof_job = max(flops_step / world / (pk["bf16_sustained"] * 1e12), 0.0)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(args.config, cfg), "l2": "256 MB buffer written between timed steps",
                       "schedule": "single GPU" if world == 1 else lvx.attn._schedule(None, q),
                       "timing": "CUDA events per step on the launch stream, summed; max over ranks"},
            "ms_per_layer": ms_per_step, "tflops_per_gpu": value / world,
            "frac_of_tensor_roofline": (roof_job * 1e3) / ms_per_step, "wall_ms": wall_ms,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
