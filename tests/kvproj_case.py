"""Runs lvx_kv_project once (or a few times) at the Llama-3.2-Vision projection shape -- hidden 4096, 8 KV heads --
on S synthetic visual tokens and prints its event-timed duration: the small, self-ending workload to put under ncu.

    python tests/kvproj_case.py [S] [ITERS]          (S = 51232: one rank's share of 409,856 tokens at 8 ranks;
                                                      X is 420 MB, larger than L2)
"""
import sys, os, torch
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from lv_xattn_b200 import ops, _lib
S = int(sys.argv[1]) if len(sys.argv) > 1 else 51232
it = int(sys.argv[2]) if len(sys.argv) > 2 else 1
dev = torch.device("cuda", 0)
g = torch.Generator(device=dev).manual_seed(0)
x = torch.empty(1, S, 4096, device=dev).normal_(0, 1, generator=g).bfloat16()
wk = torch.empty(1024, 4096, device=dev).normal_(0, 0.02, generator=g).bfloat16()
wv = torch.empty(1024, 4096, device=dev).normal_(0, 0.02, generator=g).bfloat16()
nw = torch.ones(128, device=dev).bfloat16()
for _ in range(it):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(); k, v, r = ops.kv_project(x, wk, wv, nw, 1e-5, 8); b.record(); torch.cuda.synchronize()
ms = a.elapsed_time(b)
print(f"kv_project S={S}: {ms:.3f} ms {2*2*S*4096*1024/ms/1e9:.0f} TFLOP/s status {_lib.device_status()}")
