#!/usr/bin/env python
"""Benchmark of the sequence-parallel cross-attention layer (forward + backward), one JSON line on rank 0.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 1|2|3|5]

Workloads (N = 1..8 ranks, total work fixed => strong scaling; Q/dO and K/V are sharded evenly by sequence over
the ranks, rank r takes the r-th slice, reference test.py:164-178; inputs are seeded synthetic tensors with the
reference benchmark's distributions, test.py:101-107: q,k,v ~ N(0,0.5^2), dO ~ N(0,1)):
  config 2 (default, the headline)  B=1, Hq=32, Hkv=8, D=128, Sq=2048 text queries, Skv=131072 visual keys, bf16
  config 1  the reference's CPU-runnable correctness shape: Sq=512, Skv=8192, fp32 (exact FP32-FMA kernels)
  config 5  long-visual stress: B=2, Sq=256, Skv=1048576, key padding to 1048576 / 786432 valid keys, bf16
  config 4  end-to-end training step (forward, loss, backward, gradient all-reduce; no optimizer, as in the reference's
            driver test_llama3.py:710-737) of a random-init Llama-3.2-11B-Vision-shaped text decoder: 40 layers, gated
            cross-attention at 3,8,...,38, hidden 4096, FFN 14336, vocab 128256, 2048 tokens, visual states
            [1,262144,4096]; both Hugging Face hooks installed, text and visual sequences sharded over the ranks
  config 3  Llama-3.2-11B-Vision-shaped cross-attention block (hidden 4096, per-head RMSNorm on q and k, q/k/v/o
            projections N(0,0.02^2), states [1,409856,4096], text [1,1024,4096], bf16) through the
            patch_cross_attention_forward hook with K/V recomputed in backward

A step = one forward + one backward through lv_xattn_b200._attn_forward/_attn_backward (config 3: through the
hooked module).
  value   whole-job algorithmic TFLOP/s (3.5 * 4*Hq*D*Sq*sum_b Skv_valid[b] per step over all ranks; config 3 adds
          the projection GEMMs), inputs resident in HBM, device time from CUDA events summed over the K steps,
          max over ranks
  e2e     the same through lv_xattn_b200.HostStreamedAttention.step with HOST (pinned) inputs and outputs:
          H2D of q,k,v,dO and D2H of o,dq,dk,dv inside the timed region. Consecutive steps are pipelined (the
          copy of step i+1's inputs and the drain of step i's results overlap the kernels), timed from before the
          first copy to after the last result has landed; `latency_ms_per_step` is one step alone
  roofline  the backward block kernel: algorithmic FLOPs of its launches / its event-timed duration, against
          the measured bf16 tensor peak; `hbm_gbs` = algorithmic K/V/dK/dV + Q-side bytes per step / step time
  parity  after the timed region every rank recomputes one KV group of the full problem in fp32 on its GPU
          (oracle.group_fwd_bwd on inputs regenerated from the seeds of all ranks) and compares its own shard of
          O, lse, dQ, dK, dV; max over ranks; a failure makes the run exit non-zero
          (the reference's benchmark checks every shard the same way, test.py:192, :210-212)
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
    1: dict(B=1, Hq=32, Hkv=8, D=128, Sq=512, Skv=8192, dtype="f32", valid=None),
    2: dict(B=1, Hq=32, Hkv=8, D=128, Sq=2048, Skv=131072, dtype="bf16", valid=None),
    3: dict(B=1, Hq=32, Hkv=8, D=128, Sq=1024, Skv=409856, dtype="bf16", valid=None, hidden=4096, layer=True),
    4: dict(B=1, Hq=32, Hkv=8, D=128, Sq=2048, Skv=262144, dtype="bf16", valid=None, hidden=4096, decoder=True,
            layers=40, cross_layers=list(range(3, 40, 5)), ffn=14336, vocab=128256),
    5: dict(B=2, Hq=32, Hkv=8, D=128, Sq=256, Skv=1048576, dtype="bf16", valid=[1048576, 786432]),
}
TORCH_DTYPE = {"bf16": torch.bfloat16, "f32": torch.float32}
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
    """Seeded full-tensor statistics, generated shard-wise on the device (each rank only its slices; the
    generator is seeded by (seed, rank), so any rank can regenerate any other rank's shard)."""
    B, Hq, Hkv, D, Sq, Skv = (cfg[n] for n in ("B", "Hq", "Hkv", "D", "Sq", "Skv"))
    g = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    Sl, Kl = Sq // world, Skv // world
    q = torch.empty(B, Hq, Sl, D, device=device).normal_(0, 0.5, generator=g).to(dtype)
    k = torch.empty(B, Hkv, Kl, D, device=device).normal_(0, 0.5, generator=g).to(dtype)
    v = torch.empty(B, Hkv, Kl, D, device=device).normal_(0, 0.5, generator=g).to(dtype)
    do = torch.empty(B, Hq, Sl, D, device=device).normal_(0, 1.0, generator=g).to(dtype)
    return q, k, v, do


def valid_list(cfg):
    return cfg["valid"] if cfg["valid"] is not None else [cfg["Skv"]] * cfg["B"]


def cpu_attention_sample(cfg, threads, heads):
    """The CPU oracle on a bounded sample of the workload: `heads` query heads of the first batch entry (one head
    per pass so that a [Sq, Skv] fp32 score matrix stays near 1 GiB), all Sq queries, all valid keys.
    Returns (TFLOP/s, seconds, description)."""
    from oracle import attention_oracle as orc
    Hq, D, Sq = cfg["Hq"], cfg["D"], cfg["Sq"]
    skv = valid_list(cfg)[0]
    torch.set_num_threads(threads)
    q, k, v, do = orc.make_inputs(1, heads, 1, Sq, skv, D, 1, torch.float32)
    t0 = time.perf_counter()
    for h in range(heads):
        orc.attention_fwd_bwd(q[:, h:h + 1], k, v, do[:, h:h + 1], 1.0 / math.sqrt(D))
    dt = time.perf_counter() - t0
    f_fwd, f_bwd = orc.flops_fwd_bwd(1, heads, D, Sq, skv)
    tot = sum(orc.flops_fwd_bwd(cfg["B"], Hq, D, Sq, valid_list(cfg)))
    desc = (f"fp32 torch CPU fwd+bwd (reference test.py:129-156 math), {heads} of {Hq} query heads of batch entry 0, "
            f"Sq={Sq} Skv={skv} ({(f_fwd + f_bwd) / tot:.4f} of the workload's FLOPs)")
    return (f_fwd + f_bwd) / dt / 1e12, dt, desc


def cpu_sample_heads(cfg, big):
    """Heads per CPU sample, sized for roughly 10-30 s of host work."""
    per_head = cfg["Sq"] * valid_list(cfg)[0]
    base = 2048 * 131072
    n = (16 if big else 4) * base / per_head
    return int(max(1, min(cfg["Hq"], round(n))))


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals = []
    for i in range(args.warmup + args.steps):
        tf, dt, desc = cpu_attention_sample(cfg, threads, cpu_sample_heads(cfg, False))
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
    s = (f"config{cid}: xattn fwd+bwd B={cfg['B']} Hq={cfg['Hq']} Hkv={cfg['Hkv']} D={cfg['D']} Sq={cfg['Sq']} "
         f"Skv={cfg['Skv']} {cfg['dtype']}")
    if cfg["valid"] is not None:
        s += f" kv_valid_len={cfg['valid']}"
    if cfg.get("layer"):
        s += f" Llama-3.2-11B-Vision cross-attention block (hidden {cfg['hidden']}, K/V recomputed in backward)"
    if cfg.get("decoder"):
        s += (f" per cross layer; {cfg['layers']}-layer Llama-3.2-11B-Vision-shaped text decoder, cross-attention layers "
              f"{cfg['cross_layers']}, hidden {cfg['hidden']}, training step without optimizer")
    return s + ", Q and K/V sharded by sequence"


def parity_probe(cfg, rank, world, seed, dev, dtype, outs, scale):
    """This rank's shard of (o, L, dq, dk, dv) against one KV group of the full problem recomputed in fp32 on the
    GPU from the regenerated inputs of all ranks. Returns a dict of max-abs errors, the largest relative
    Frobenius error and ok (absolute bars: 16-bit 2e-2 / lse 1e-3, fp32 1e-4; relative: Frobenius <= 1e-2
    (fp32 1e-4), max error <= 5 % of max|ref|)."""
    from oracle import attention_oracle as orc
    o, L, dq, dk, dv = outs
    B, Hq, Hkv, Sq, Skv = (cfg[n] for n in ("B", "Hq", "Hkv", "Sq", "Skv"))
    g = Hq // Hkv
    b, hk = rank % B, (rank // B) % Hkv
    hs = slice(hk * g, (hk + 1) * g)
    qs, ks, vs, dos = [], [], [], []
    for s in range(world):                     # every rank's shard of this group, in rank order = sequence order
        q_s, k_s, v_s, do_s = gen_inputs(cfg, s, world, seed, dev, dtype)
        qs.append(q_s[b, hs].clone())
        dos.append(do_s[b, hs].clone())
        ks.append(k_s[b, hk].clone())
        vs.append(v_s[b, hk].clone())
        del q_s, k_s, v_s, do_s
    qf, dof = torch.cat(qs, 1), torch.cat(dos, 1)
    kf, vf = torch.cat(ks, 0), torch.cat(vs, 0)
    o_r, lse_r, dq_r, dk_r, dv_r = orc.group_fwd_bwd(qf, kf, vf, dof, scale, valid_list(cfg)[b])
    Sl, Kl = Sq // world, Skv // world
    rq, rk = slice(rank * Sl, (rank + 1) * Sl), slice(rank * Kl, (rank + 1) * Kl)
    fp32 = dtype == torch.float32
    abs_tol, fro_tol, lse_tol = (1e-4, 1e-4, 1e-4) if fp32 else (2e-2, 1e-2, 1e-3)
    res, ok, rel_max = {}, True, 0.0
    lse_got, lse_ref = L.view(B, Hq, Sl)[b, hs], lse_r[:, rq]
    fin = torch.isfinite(lse_ref)
    ok = ok and bool(torch.equal(torch.isfinite(lse_got), fin))
    res["lse"] = (lse_got[fin] - lse_ref[fin]).abs().max().item() if fin.any() else 0.0
    ok = ok and res["lse"] <= lse_tol
    for name, got, ref in (("o", o[b, hs], o_r[:, rq]), ("dq", dq[b, hs], dq_r[:, rq]), ("dk", dk[b, hk], dk_r[rk]),
                           ("dv", dv[b, hk], dv_r[rk])):
        d = got.float() - ref
        ma, rn, rm = d.abs().max().item(), ref.norm().item(), ref.abs().max().item()
        fro = d.norm().item() / rn if rn > 0 else (0.0 if ma == 0 else float("inf"))
        res[name] = ma
        rel_max = max(rel_max, fro)
        ok = ok and bool(torch.isfinite(got.float()).all()) and ma <= abs_tol and fro <= fro_tol and ma <= 0.05 * rm + 1e-30
    res["rel_max"] = rel_max
    res["ok"] = bool(ok)
    res["checked"] = f"KV group (batch {b}, kv head {hk}) of every rank's shard, all rows and keys, vs fp32 on the GPU"
    return res


def layer_flops(cfg):
    """(attention core, projections) algorithmic FLOPs of one forward + backward of the cross-attention block:
    core 3.5 * 4*Hq*D*Sq*Skv; K and V projections 2*Skv*hidden*Hkv*D each, run in forward, again in the backward
    recompute, and once more for their weight gradients (the states need no gradient); q and o projections
    forward, input gradient and weight gradient, q once more in the recompute."""
    Hq, Hkv, D, Sq, Skv, hid = (cfg[n] for n in ("Hq", "Hkv", "D", "Sq", "Skv", "hidden"))
    core = 3.5 * 4.0 * Hq * D * Sq * Skv
    kv = 3 * 2 * (2.0 * Skv * hid * Hkv * D)
    qo = (4 + 3) * (2.0 * Sq * hid * Hq * D)
    return core, kv + qo


def run_layer(args, cfg, rank, world, local, dev):
    """Config 3: the Llama-3.2-11B-Vision-shaped cross-attention block through patch_cross_attention_forward
    (random-init weights N(0,0.02^2), RMSNorm weights 1, synthetic N(0,1) states and hidden states generated
    shard-wise from (seed, rank) -- they stand in for the reference's real-model run, test_llama3.py:657-770).
    Returns False when the parity probe fails."""
    import lv_xattn_b200 as lvx
    from lv_xattn_b200 import _lib, hf_patch, ops
    from oracle import attention_oracle as orc
    from transformers.models.mllama import modeling_mllama as mllama

    Hq, Hkv, D, Sq, Skv, hid = (cfg[n] for n in ("Hq", "Hkv", "D", "Sq", "Skv", "hidden"))
    Sl, Kl = Sq // world, Skv // world
    mcfg = mllama.MllamaTextConfig(hidden_size=hid, num_attention_heads=Hq, num_key_value_heads=Hkv,
                                   num_hidden_layers=4, intermediate_size=14336, vocab_size=128256)
    mcfg._attn_implementation = "eager"
    torch.manual_seed(1234)                               # the same weights on every rank
    with torch.device("meta"):
        mod = mllama.MllamaTextCrossAttention(mcfg, layer_idx=3)
    mod = mod.to_empty(device=dev).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(1234)
    with torch.no_grad():
        for name, p in mod.named_parameters():
            if "norm" in name:
                p.fill_(1.0)
            else:
                p.copy_(torch.empty(p.shape, device=dev).normal_(0, 0.02, generator=gw))
    mod.forward = hf_patch.patch_cross_attention_forward("lv_xattn").__get__(mod)

    def gen(r):
        g = torch.Generator(device=dev).manual_seed(3000 + r)
        x = torch.empty(1, Sl, hid, device=dev).normal_(0, 1, generator=g).bfloat16()
        st = torch.empty(1, Kl, hid, device=dev).normal_(0, 1, generator=g).bfloat16()
        go = torch.empty(1, Sl, hid, device=dev).normal_(0, 1, generator=g).bfloat16()
        return x, st, go

    x, states, gout = gen(rank)
    x.requires_grad_(True)
    hf_patch.set_global_cross_attention_states(states)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def step():
        x.grad = None
        for p in mod.parameters():
            p.grad = None
        out, _ = mod(x)
        out.backward(gout)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        evs = []
        for _ in range(steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            evs.append((a, b))
        barrier()
        t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t[0].item()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    ops.set_profiling(True)
    ops.launch_count = 0
    n_before = len(sampler.samples)
    total_ms = timed(step, args.steps, 0)
    sampler.samples = sampler.samples[n_before:] or sampler.samples[-1:]
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.launch_count
    prof = ops.take_profile()
    ops.set_profiling(False)
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"device status word {status:#x}: a bounded wait ran out")
    ms = total_ms / args.steps
    core, proj = layer_flops(cfg)
    pk = peaks()
    bwd_ms, fwd_ms = sum(prof["bwd"]) / args.steps, sum(prof["fwd"]) / args.steps
    proj_ms = sum(prof.get("proj", [])) / args.steps
    achieved = (core * 2.5 / 3.5 / world) / (bwd_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "bwd_kernel", "achieved": achieved, "peak": pk["bf16_sustained"],
                "unit": "TFLOP/s", "frac": achieved / pk["bf16_sustained"],
                "peak_source": f"{pk['source']} (sustained cuBLAS bf16)", "traffic": None,
                "bwd_kernel_ms_per_step": bwd_ms, "fwd_kernel_ms_per_step": fwd_ms,
                "kv_projection_kernel_ms_per_step": proj_ms,
                "attention_core_ms_per_step": bwd_ms + fwd_ms,
                "attention_core_tflops_per_gpu": core / world / ((bwd_ms + fwd_ms) * 1e-3) / 1e12}

    # ---- parity probe: the block in fp32 on the GPU (attention through the oracle's group form), all ranks' rows ----
    parity = None
    if not args.no_parity:
        out = step().detach()
        dx = x.grad.detach().clone()
        torch.cuda.synchronize()
        xs, sts, gos = zip(*(gen(r) for r in range(world)))
        xf = torch.cat(xs, 1)[0].float().requires_grad_(True)
        W = {n: p.detach().float() for n, p in mod.named_parameters()}
        eps = mod.q_norm.variance_epsilon if hasattr(mod.q_norm, "variance_epsilon") else mcfg.rms_norm_eps
        tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False

        def rms(t, w):
            return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w

        qf = rms((xf @ W["q_proj.weight"].t()).view(Sq, Hq, D), W["q_norm.weight"]).transpose(0, 1)    # [Hq,Sq,D]
        kf = torch.empty(Hkv, Skv, D, device=dev)
        vf = torch.empty(Hkv, Skv, D, device=dev)
        for r in range(world):                                  # shard by shard: the fp32 states are 6.7 GB in all
            sf = sts[r][0].float()
            kf[:, r * Kl:(r + 1) * Kl] = rms((sf @ W["k_proj.weight"].t()).view(Kl, Hkv, D), W["k_norm.weight"]).transpose(0, 1)
            vf[:, r * Kl:(r + 1) * Kl] = (sf @ W["v_proj.weight"].t()).view(Kl, Hkv, D).transpose(0, 1)
            del sf
        gof = torch.cat(gos, 1)[0].float()
        d_attn = (gof @ W["o_proj.weight"]).view(Sq, Hq, D).transpose(0, 1)                             # dO per head
        g = Hq // Hkv
        o_ref = torch.empty(Hq, Sq, D, device=dev)
        dq_ref = torch.empty(Hq, Sq, D, device=dev)
        for hk in range(Hkv):
            hs = slice(hk * g, (hk + 1) * g)
            o_g, _, dq_g, _, _ = orc.group_fwd_bwd(qf[hs].detach(), kf[hk], vf[hk], d_attn[hs], D ** -0.5)
            o_ref[hs], dq_ref[hs] = o_g, dq_g
        out_ref = o_ref.transpose(0, 1).reshape(Sq, Hq * D) @ W["o_proj.weight"].t()
        (dx_ref,) = torch.autograd.grad(qf, xf, dq_ref)
        torch.backends.cuda.matmul.allow_tf32 = tf32
        rows = slice(rank * Sl, (rank + 1) * Sl)
        parity, ok = {}, True
        for name, got, ref in (("out", out[0], out_ref[rows]), ("dx", dx[0], dx_ref[rows])):
            d = got.float() - ref
            fro = d.norm().item() / ref.norm().item()
            parity[name] = d.abs().max().item()
            parity[name + "_rel"] = fro
            ok = ok and bool(torch.isfinite(got.float()).all()) and fro <= 2e-2
        parity["rel_max"] = max(parity["out_rel"], parity["dx_rel"])
        parity["ok"] = bool(ok)
        parity["checked"] = ("block output and hidden-state gradient of this rank's rows vs the whole block in fp32 on "
                             "the GPU (relative Frobenius error <= 2e-2: two bf16 GEMMs and two bf16 roundings deep)")
        if world > 1:
            keys = ["out", "dx", "out_rel", "dx_rel", "rel_max"]
            t = torch.tensor([parity[n] for n in keys] + [0.0 if parity["ok"] else 1.0], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            for n, v_ in zip(keys, t.tolist()):
                parity[n] = v_
            parity["ok"] = t[-1].item() == 0.0
        del xs, sts, gos, kf, vf, qf, o_ref, dq_ref
        torch.cuda.empty_cache()

    # ---- end to end: hidden states, visual states and upstream gradient start in pinned host memory ----
    e2e = None
    if not args.no_e2e:
        hx, hst, hgo = (t.detach().cpu().pin_memory() for t in (x, states, gout))
        hout, hdx = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()

        def step_e2e():
            nonlocal x, states, gout
            x = hx.to(dev, non_blocking=True).requires_grad_(True)
            states = hst.to(dev, non_blocking=True)
            gout = hgo.to(dev, non_blocking=True)
            hf_patch.set_global_cross_attention_states(states)
            out_ = step()
            hout.copy_(out_.detach(), non_blocking=True)
            hdx.copy_(x.grad, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        e_steps = max(1, min(args.steps, 5))
        e_ms = timed(step_e2e, e_steps, 1)
        h2d = sum(t.numel() * t.element_size() for t in (hx, hst, hgo))
        d2h = sum(t.numel() * t.element_size() for t in (hout, hdx))
        e2e = {"value": (core + proj) / (e_ms / e_steps * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e_ms / e_steps,
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e_steps}
    hf_patch.clear_global_cross_attention_states()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tf, dt, desc = cpu_attention_sample(cfg, threads, cpu_sample_heads(cfg, True))
        cpu = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc + " (attention core only)",
               "seconds": dt}

    if rank == 0:
        value = (core + proj) / (ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name(args.config, cfg), "l2": "256 MB buffer written between timed steps",
                       "schedule": "single GPU" if world == 1 else lvx.attn._schedule(None, x),
                       "flops": {"attention_core": core, "projections": proj},
                       "timing": "CUDA events per step on the launch stream, summed; max over ranks"},
            "ms_per_layer": ms, "tflops_per_gpu": value / world,
            "frac_of_tensor_roofline": ((core + proj) / world / (pk["bf16_sustained"] * 1e12) * 1e3) / ms,
            "roofline": roofline, "parity": parity, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    return parity is None or parity["ok"]


def run_decoder(args, cfg, rank, world, local, dev):
    """Config 4: a training step of the whole text decoder with both hooks installed (hf_patch.install_hooks, as the
    reference assigns them at test_llama3.py:666-667). Random-init weights N(0,0.02^2), norm weights 1, the
    cross-attention gates 0.25 (the stock init of 0 would switch the cross-attention layers off), token ids and labels
    uniform, visual states N(0,1) generated shard-wise: synthetic stand-ins for the reference's real-model run
    (test_llama3.py:657-770). The weights are replicated; every rank differentiates its shard of the sequence and the
    gradients are summed with an NCCL all-reduce inside the timed step. Returns False when the loss is not finite."""
    import lv_xattn_b200 as lvx
    from lv_xattn_b200 import _lib, hf_patch, ops
    from transformers.models.mllama import modeling_mllama as mllama

    Hq, Hkv, D, Sq, Skv, hid = (cfg[n] for n in ("Hq", "Hkv", "D", "Sq", "Skv", "hidden"))
    layers = args.layers or cfg["layers"]
    cross = [i for i in cfg["cross_layers"] if i < layers]
    Sl, Kl = Sq // world, Skv // world
    mcfg = mllama.MllamaTextConfig(hidden_size=hid, num_attention_heads=Hq, num_key_value_heads=Hkv,
                                   num_hidden_layers=layers, intermediate_size=cfg["ffn"], vocab_size=cfg["vocab"],
                                   cross_attention_layers=cross, max_position_embeddings=max(Sq, 4096), pad_token_id=0)
    mcfg._attn_implementation = "eager"
    with torch.device("meta"):
        model = mllama.MllamaForCausalLM(mcfg)
    model = model.to_empty(device=dev).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(4321)          # the same weights on every rank
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "gate" in name:
                p.fill_(0.25)
            elif "norm" in name:
                p.fill_(1.0)
            else:
                p.copy_(torch.empty(p.shape, device=dev).normal_(0, 0.02, generator=gw))
        for name, b in model.named_buffers():               # rotary tables were allocated on the meta device
            if "inv_freq" in name:
                rope = mllama.MllamaRotaryEmbedding(mcfg, device=dev)
                b.copy_(rope.inv_freq)
    n_params = sum(p.numel() for p in model.parameters())
    hf_patch.install_hooks("lv_xattn")
    g = torch.Generator(device=dev).manual_seed(5000 + rank)
    ids = torch.randint(1, cfg["vocab"], (1, Sl), device=dev, generator=g)
    labels = torch.randint(1, cfg["vocab"], (1, Sl), device=dev, generator=g)
    states = torch.empty(1, Kl, hid, device=dev).normal_(0, 1, generator=g).bfloat16()
    pos = (torch.arange(Sl, device=dev) + rank * Sl)[None]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    params = [p for p in model.parameters()]

    def step(ids_=None, states_=None):
        for p in params:
            p.grad = None
        h = model.model(input_ids=ids if ids_ is None else ids_, position_ids=pos, use_cache=False,
                        cross_attention_states=states if states_ is None else states_).last_hidden_state
        logits = model.lm_head(h).float()
        loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), labels.view(-1), reduction="sum") / Sq
        loss.backward()
        if world > 1:                                  # replicated weights: sum the ranks' gradients
            works = [dist.all_reduce(p.grad, async_op=True) for p in params if p.grad is not None]
            for w in works:
                w.wait()
        return loss.detach()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        evs = []
        for _ in range(steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            evs.append((a, b))
        barrier()
        t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t[0].item()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    ops.set_profiling(True)
    ops.launch_count = 0
    n_before = len(sampler.samples)
    total_ms = timed(step, args.steps, 0)
    sampler.samples = sampler.samples[n_before:] or sampler.samples[-1:]
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.launch_count
    prof = ops.take_profile()
    ops.set_profiling(False)
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"device status word {status:#x}: a bounded wait ran out")
    ms = total_ms / args.steps
    loss = step()
    if world > 1:
        dist.all_reduce(loss)
    loss_v = loss.item()
    nc = len(cross)
    core = nc * 3.5 * 4.0 * Hq * D * Sq * Skv
    proj = nc * 3 * 2 * (2.0 * Skv * hid * Hkv * D)
    dense = 6.0 * (n_params - cfg["vocab"] * hid) * Sq            # embedding lookup does no FLOPs; the head does
    self_attn = (layers - nc) * 3.5 * 4.0 * Hq * D * Sq * Sq / 2
    flops = core + proj + dense + self_attn
    pk = peaks()
    bwd_ms, fwd_ms = sum(prof["bwd"]) / args.steps, sum(prof["fwd"]) / args.steps
    proj_ms = sum(prof.get("proj", [])) / args.steps
    achieved = (core * 2.5 / 3.5 / world) / (bwd_ms * 1e-3) / 1e12 if bwd_ms > 0 else 0.0
    roofline = {"bound": "tensor", "kernel": "bwd_kernel", "achieved": achieved, "peak": pk["bf16_sustained"],
                "unit": "TFLOP/s", "frac": achieved / pk["bf16_sustained"],
                "peak_source": f"{pk['source']} (sustained cuBLAS bf16)", "traffic": None,
                "bwd_kernel_ms_per_step": bwd_ms, "fwd_kernel_ms_per_step": fwd_ms,
                "kv_projection_kernel_ms_per_step": proj_ms,
                "cross_attention_core_ms_per_step": bwd_ms + fwd_ms,
                "ms_per_cross_layer_core": (bwd_ms + fwd_ms) / max(nc, 1)}
    parity = {"loss": loss_v, "ok": bool(math.isfinite(loss_v)), "rel_max": None,
              "checked": ("loss finite (ln(vocab) = %.3f for random weights). Sharded-versus-unsharded parity of the whole "
                          "decoder through both hooks is tests/test_decoder_cpu.py (two gloo ranks, every parameter's "
                          "gradient); the hooks with the real kernels are tests/test_gpu_hf_patch.py and "
                          "tests/test_gpu_multi.py; no reference numbers exist for this configuration" % math.log(cfg["vocab"]))}

    e2e = None
    if not args.no_e2e:
        hids, hst = ids.cpu().pin_memory(), states.cpu().pin_memory()
        hloss = torch.empty((), dtype=torch.float32).pin_memory()

        def step_e2e():
            l_ = step(hids.to(dev, non_blocking=True), hst.to(dev, non_blocking=True))
            hloss.copy_(l_, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        e_steps = max(1, min(args.steps, 3))
        e_ms = timed(step_e2e, e_steps, 1)
        e2e = {"value": flops / (e_ms / e_steps * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e_ms / e_steps,
               "h2d_bytes_per_step": world * (hids.numel() * 8 + hst.numel() * 2), "d2h_bytes_per_step": world * 4,
               "steps": e_steps}
    hf_patch.uninstall_hooks()
    hf_patch.clear_global_cross_attention_states()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tf, dt, desc = cpu_attention_sample(cfg, threads, cpu_sample_heads(cfg, True))
        cpu = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc + " (cross-attention core only)",
               "seconds": dt}
    if rank == 0:
        value = flops / (ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name(args.config, cfg), "layers": layers, "parameters": n_params,
                       "l2": "256 MB buffer written between timed steps",
                       "schedule": "single GPU" if world == 1 else lvx.attn._schedule(None, states),
                       "flops": {"cross_attention_core": core, "kv_projections": proj, "dense_layers_and_head": dense,
                                 "self_attention": self_attn},
                       "timing": "CUDA events per step on the launch stream, summed; max over ranks"},
            "ms_per_layer": (bwd_ms + fwd_ms + proj_ms) / max(nc, 1), "tflops_per_gpu": value / world,
            "frac_of_tensor_roofline": (flops / world / (pk["bf16_sustained"] * 1e12) * 1e3) / ms,
            "roofline": roofline, "parity": parity, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    return parity["ok"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS))
    ap.add_argument("--layers", type=int, default=None, help="config 4 only: fewer decoder layers (a smoke run)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=8,
                    help="K/V chunks of the host-streamed step timed on its own (latency_ms_per_step)")
    ap.add_argument("--e2e-pipeline-chunks", type=int, default=4,
                    help="K/V chunks per step of the pipelined end-to-end loop (the copies hide behind the "
                         "neighbouring steps there; chunks only shorten the first step's copy-in and the last "
                         "step's copy-out, which the timed region includes)")
    ap.add_argument("--attention", default="lv_xattn", choices=["lv_xattn", "ring"],
                    help="lv_xattn: the query side rotates, K/V resident (the product path); ring: the K/V-rotating "
                         "ring-attention baseline on the same kernels (reference ring/attn.py), for comparison")
    ap.add_argument("--schedule", default=None, help="LV-XAttn exchange schedule (default: LVX_SCHEDULE or auto)")
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
    from oracle import attention_oracle as orc  # FLOP formula and the parity probe's fp32 reference

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        lvx.initialize_distributed("nccl")

    if cfg.get("decoder"):
        ok = run_decoder(args, cfg, rank, world, local, dev)
        if world > 1:
            dist.destroy_process_group()
        if not ok:
            raise SystemExit("config 4: loss not finite")
        return
    if cfg.get("layer"):
        ok = run_layer(args, cfg, rank, world, local, dev)
        if world > 1:
            dist.destroy_process_group()
        if not ok:
            raise SystemExit("parity probe failed")
        return

    B, Hq, Hkv, D, Sq, Skv = (cfg[n] for n in ("B", "Hq", "Hkv", "D", "Sq", "Skv"))
    dtype = TORCH_DTYPE[cfg["dtype"]]
    valid = cfg["valid"]
    scale = 1.0 / math.sqrt(D)
    seed = 1
    q, k, v, do = gen_inputs(cfg, rank, world, seed, dev, dtype)
    f_fwd, f_bwd = orc.flops_fwd_bwd(B, Hq, D, Sq, valid_list(cfg))
    flops_step = f_fwd + f_bwd
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB L2

    if args.attention == "ring":
        from lv_xattn_b200 import ring as impl
        sched_kw = {}
    else:
        impl = lvx
        sched_kw = {"schedule": args.schedule} if args.schedule else {}

    def step_device():
        _, _, _, o, L = impl._attn_forward(q, k, v, False, scale, None, kv_valid_len=valid, **sched_kw)
        return impl._attn_backward(do, q, k, v, o, L, False, scale, None, "flash", kv_valid_len=valid, **sched_kw) + (o, L)

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
    # dominant kernel: the backward block. Its launches of one step together do this rank's share of f_bwd
    # (with key padding the shares differ; the job-wide mean is used).
    bwd_ms_step = sum(prof["bwd"]) / args.steps
    fwd_ms_step = sum(prof["fwd"]) / args.steps
    achieved = (f_bwd / world) / (bwd_ms_step * 1e-3) / 1e12
    peak = pk["bf16_sustained"]
    es = 2 if dtype != torch.float32 else 4
    # algorithmic HBM bytes of one step on one rank: K and V read by forward and by backward, dK and dV written,
    # Q/dO/O/dQ-side tensors of all query blocks once each way
    kv_bytes = 2 * sum(min(max(n - rank * (Skv // world), 0), Skv // world) for n in valid_list(cfg)) * Hkv * D * es
    q_bytes = B * Hq * Sq * D * es
    alg_bytes = 2 * kv_bytes + kv_bytes + 6 * q_bytes
    roofline = {"bound": "tensor", "kernel": "bwd_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "peak_source": f"{pk['source']} (sustained cuBLAS bf16)",
                # DRAM bytes per launch, from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum) of one
                # launch at Sq=2048, Skv=32768: 324.5 MB, of which 268.4 MB is K,V in and dK,dV out (scales with
                # this rank's key rows) and 56 MB is Q, dO and dQ (all query blocks pass through every rank)
                "traffic": (268.4e6 * (B * Skv / world) / 32768 + 56e6 * (B * Sq / 2048)) if dtype != torch.float32 else None,
                "traffic_source": "ncu capture at Skv=32768 scaled by key rows",
                "bwd_kernel_ms_per_step": bwd_ms_step, "fwd_kernel_ms_per_step": fwd_ms_step,
                "fwd_achieved": (f_fwd / world) / (fwd_ms_step * 1e-3) / 1e12,
                "hbm_gbs": alg_bytes / (ms_per_step * 1e-3) / 1e9, "hbm_peak_gbs": pk["hbm_gbs"],
                "launches_per_step": {"fwd": len(prof["fwd"]) // args.steps, "bwd": len(prof["bwd"]) // args.steps}}
    if dtype == torch.float32:
        roofline["note"] = ("fp32 inputs run the exact FP32-FMA kernels (correctness configuration); the fraction is "
                            "quoted against the bf16 tensor peak for comparability and is expected to be small")

    # ---- parity probe (outside every timed region) --------------------------------------------------
    parity = None
    if not args.no_parity:
        dq_, dk_, dv_, o_, L_ = step_device()
        torch.cuda.synchronize()
        parity = parity_probe(cfg, rank, world, seed, dev, dtype, (o_, L_, dq_, dk_, dv_), scale)
        del dq_, dk_, dv_, o_, L_
        if world > 1:
            keys = ["o", "lse", "dq", "dk", "dv", "rel_max"]
            t = torch.tensor([parity[n] for n in keys] + [0.0 if parity["ok"] else 1.0], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            for n, x in zip(keys, t.tolist()):
                parity[n] = x
            parity["ok"] = t[-1].item() == 0.0
            parity["checked"] = "on every rank: one " + parity["checked"]
        torch.cuda.empty_cache()

    # ---- end-to-end run: host (pinned) inputs, results read back ------------------------------------
    e2e = None
    if not args.no_e2e and args.attention == "lv_xattn":
        hq, hk, hv, hdo = (t.cpu().pin_memory() for t in (q, k, v, do))
        ho, hdq = torch.empty_like(hq).pin_memory(), torch.empty_like(hq).pin_memory()
        hdk, hdv = torch.empty_like(hk).pin_memory(), torch.empty_like(hv).pin_memory()

        streamer = lvx.HostStreamedAttention(dev, chunks=args.e2e_chunks)

        def step_e2e():
            streamer.step(hq, hk, hv, hdo, scale, ho, hdq, hdk, hdv, kv_valid_len=valid)

        # latency of one step on its own: copy in, compute, copy out, nothing from a neighbouring step overlapped
        # (median of three, each timed on its own after two untimed ones: a single step is short enough for one
        # stray host stall to double a mean)
        for _ in range(2):
            step_e2e()
        lats = []
        for _ in range(3):
            flush.zero_()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step_e2e()
            b.record()
            torch.cuda.synchronize()
            lats.append(a.elapsed_time(b))
        t = torch.tensor([sorted(lats)[1]], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        lat_ms = t[0].item()

        # throughput over consecutive steps, as a training loop runs them: the inputs of step i+1 are copied while
        # step i computes and the results of step i drain while step i+1 runs. Every step's inputs cross the host
        # link inside the timed region and every step's results are back in host memory before it ends.
        e_steps = max(2, min(args.steps, 20))
        del streamer                                  # its device buffers go back to the allocator
        torch.cuda.empty_cache()
        streamer = lvx.HostStreamedAttention(dev, chunks=args.e2e_pipeline_chunks)
        streamer.step(hq, hk, hv, hdo, scale, ho, hdq, hdk, hdv, kv_valid_len=valid)      # untimed: allocates
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        streamer.prefetch(hq, hk, hv, hdo)
        for i in range(e_steps):
            flush.zero_()
            if i + 1 < e_steps:
                streamer.prefetch(hq, hk, hv, hdo)
            streamer.step(hq, hk, hv, hdo, scale, ho, hdq, hdk, hdv, kv_valid_len=valid, wait=False)
        streamer.finish()
        b.record()
        barrier()
        t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e_ms = t[0].item()
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
        d2h = sum(t.numel() * t.element_size() for t in (ho, hdq, hdk, hdv))
        e2e = {"value": flops_step / (e_ms / e_steps * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e_ms / e_steps,
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "steps": e_steps,
               "latency_ms_per_step": lat_ms,
               "overlap": "consecutive steps pipelined over two device-side input sets, "
                          + (f"{args.e2e_pipeline_chunks} K/V chunk(s) per step; latency_ms_per_step is one step alone, "
                             f"its K/V streamed in {args.e2e_chunks} chunks" if world == 1 else
                             "each rank's whole shard per step; latency_ms_per_step is one step alone")}

    # ---- CPU baseline (rank 0, N=1 only) ----------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tf, dt, desc = cpu_attention_sample(cfg, threads, cpu_sample_heads(cfg, True))
        cpu = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc, "seconds": dt}

    if rank == 0:
        roof_job = max(flops_step / world / (pk["bf16_sustained"] * 1e12), 0.0)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
            "config": {"workload": workload_name(args.config, cfg), "l2": "256 MB buffer written between timed steps",
                       "schedule": "single GPU" if world == 1 else (
                           "ring attention baseline (K/V rotate over NCCL P2P)" if args.attention == "ring"
                           else lvx.attn._schedule(args.schedule, q)),
                       "timing": "CUDA events per step on the launch stream, summed; max over ranks"},
            "ms_per_layer": ms_per_step, "tflops_per_gpu": value / world,
            "frac_of_tensor_roofline": (roof_job * 1e3) / ms_per_step, "wall_ms": wall_ms,
            "roofline": roofline, "parity": parity, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    bad = parity is not None and not parity["ok"]
    if world > 1:
        dist.destroy_process_group()
    if bad:
        raise SystemExit(f"parity probe failed: {parity}")


if __name__ == "__main__":
    main()
