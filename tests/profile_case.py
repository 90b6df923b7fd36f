"""Runs the forward and backward block kernels once (or a few times) on a synthetic bf16 (or fp32) case and prints their
event-timed durations -- the small, self-ending workload to put under `ncu`.

    python tests/profile_case.py SQ SKV [ITERS] [B HQ HKV] [fp32]

Example (K/V = 128 MB, larger than the 126 MB L2; about 1 GB on the device):
    ncu --set full --clock-control none -k regex:bwd_kernel -c 1 -o prof python tests/profile_case.py 2048 32768
"""
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from lv_xattn_b200 import _lib, ops  # noqa: E402


def main(argv):
    sq, skv = int(argv[1]), int(argv[2])
    iters = int(argv[3]) if len(argv) > 3 else 1
    B, Hq, Hkv = (int(x) for x in argv[4:7]) if len(argv) > 6 else (1, 32, 8)
    dt = torch.float32 if "fp32" in argv[7:] else torch.bfloat16      # fp32 runs the general FP32-FMA kernels
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    q = (torch.randn(B, Hq, sq, 128, device=dev) * 0.5).to(dt)
    k = (torch.randn(B, Hkv, skv, 128, device=dev) * 0.5).to(dt)
    v = (torch.randn(B, Hkv, skv, 128, device=dev) * 0.5).to(dt)
    do = torch.randn(B, Hq, sq, 128, device=dev).to(dt)
    scale = 1.0 / math.sqrt(128.0)
    dq = torch.zeros(B, Hq, sq, 128, device=dev)
    dk = torch.empty(B, Hkv, skv, 128, device=dev, dtype=dt)   # written in the input dtype,
    dv = torch.empty_like(dk)                                               # as the step loop does
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for _ in range(iters):
        ev[0].record()
        o, lse = ops.fwd_block(q, k, v, scale)
        ev[1].record()
        delta = ops.bwd_prep(o, do)
        dq.zero_()
        ops.bwd_block(q, do, lse, delta, k, v, scale, dq, dk, dv, "final")
        ev[2].record()
        torch.cuda.synchronize()
    f = 4.0 * B * Hq * 128 * sq * skv
    tf, tb = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
    print(f"B{B} Hq{Hq} Hkv{Hkv} Sq{sq} Skv{skv}: fwd {tf:.3f} ms {f / tf / 1e9:.0f} TFLOP/s | "
          f"bwd(+prep) {tb:.3f} ms {2.5 * f / tb / 1e9:.0f} TFLOP/s | status {_lib.device_status()}")


if __name__ == "__main__":
    main(sys.argv)
