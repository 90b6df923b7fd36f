"""Generates tests/golden/ref_lvxattn_w{W}.npz from the REFERENCE's own implementation of the path.

Runs the reference's `lv_xattn._attn_forward` / `_attn_backward` (its Triton kernels under Triton's CPU
interpreter, its own step loop and P2P layer over gloo CPU ranks) on seeded inputs drawn with the reference
benchmark's protocol (test.py:101-107) and sharded as test.py:164-178. Only runs where the reference checkout
is present; the fixtures it writes are committed and are what tests/test_oracle.py reads.

    python tests/golden/make_golden.py --ref /path/to/LV-XAttn --world 1
    python tests/golden/make_golden.py --ref /path/to/LV-XAttn --world 2
    python tests/golden/make_golden.py --ref /path/to/LV-XAttn --world 4 --seed 2 --heads 1 \
        --sq-per-rank 32 --skv-per-rank 512 --tag _skv2048_seed2
    python tests/golden/make_golden.py --ref /path/to/LV-XAttn --world 2 --seed 3 --heads 1 --bias --tag _bias

Shims that touch no reference file (with --bias a fourth: the bias tensor reports is_cuda, which the reference's
backward asserts): the process group is created with gloo before
`lv_xattn.initialize_distributed()` (which then skips its NCCL init, async_communication.py:39-45),
`torch.cuda.synchronize` is a no-op, and the backward autotuner is pinned to its first config so that it
does not try to time kernels on a GPU.
"""
import argparse
import math
import os
import sys

import numpy as np


def worker(rank, world, ref, port, out_dir, seed=1, heads=2, sq_per_rank=32, skv_per_rank=128, tag="", bias=False):
    os.environ.update(TRITON_INTERPRET="1", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref)
    import torch
    import torch.distributed as dist
    torch.cuda.synchronize = lambda *a, **k: None
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import lv_xattn
    assert os.path.realpath(lv_xattn.__file__).startswith(os.path.realpath(ref)), lv_xattn.__file__
    lv_xattn.initialize_distributed()
    from lv_xattn import flash_attn_kernels as fk
    fk._bwd_kernel.configs = fk._bwd_kernel.configs[0:1]

    B, H, D = 1, heads, 128
    Sq, Skv = sq_per_rank * world, skv_per_rank * world
    torch.manual_seed(seed)                                      # test.py:101
    q = torch.empty(B, H, Sq, D, dtype=torch.float16).normal_(0.0, 0.5)
    k = torch.empty(B, H, Skv, D, dtype=torch.float16).normal_(0.0, 0.5)
    v = torch.empty(B, H, Skv, D, dtype=torch.float16).normal_(0.0, 0.5)
    do = torch.randn(B, H, Sq, D).half()
    scale = 1.0 / math.sqrt(D)

    def sl(x, n):
        return x[:, :, rank * n:(rank + 1) * n].contiguous()

    ql, dol, kl, vl = sl(q, Sq // world), sl(do, Sq // world), sl(k, Skv // world), sl(v, Skv // world)
    bias_kw, bias_full = {}, None
    if bias:
        # the reference benchmark's bias protocol (test.py:273-286): bias_func(shape, val) puts `val` on the odd key
        # columns; the shape belongs to the K/V side (local), val travels with the query block (remote). Here val
        # is 1 + home rank of the query block, so that a block that is merged with the wrong bias shows.
        class _ReportsCuda(torch.Tensor):        # the reference's backward asserts bias.is_cuda (flash_attn_kernels.py:948)
            is_cuda = property(lambda self: True)

        def bias_func(shape, val):
            b = torch.zeros([int(x) for x in shape])
            b[:, :, :, 1::2] = val
            return b.as_subclass(_ReportsCuda)
        bias_kw = dict(bias_func=bias_func,
                       local_bias_args=[torch.tensor([B, H, Sq // world, Skv // world])],
                       remote_bias_args=[torch.tensor(float(1 + rank))])
        bias_full = torch.zeros(B, 1, Sq, Skv)
        for r in range(world):
            bias_full[:, :, r * (Sq // world):(r + 1) * (Sq // world), 1::2] = float(1 + r)
    _, _, _, o, L = lv_xattn._attn_forward(ql, kl, vl, False, scale, None, **bias_kw)
    o, L = o.clone(), L.clone()
    dq, dk, dv = lv_xattn._attn_backward(dol, ql, kl, vl, o, L, False, scale, None, "flash", **bias_kw)
    outs = {"o": o, "L": L, "dq": dq, "dk": dk, "dv": dv}
    gathered = {}
    for name, t in outs.items():
        t = t.contiguous().float()
        bufs = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(bufs, t)
        gathered[name] = torch.stack(bufs).numpy()               # [W, ...] per-rank shards
    if rank == 0:
        np.savez_compressed(os.path.join(out_dir, f"ref_lvxattn_w{world}{tag}.npz"),
                            q=q.numpy(), k=k.numpy(), v=v.numpy(), do=do.numpy(), scale=np.float32(scale),
                            world=np.int32(world),
                            **({"bias": bias_full.numpy()} if bias_full is not None else {}),
                            **{f"ref_{n}": a.astype(np.float16 if n != "L" else np.float32)
                                                      for n, a in gathered.items()})
        print("wrote", f"ref_lvxattn_w{world}{tag}.npz")
    dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of the reference checkout (uw-mad-dash/LV-XAttn)")
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--port", type=int, default=29533)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--heads", type=int, default=2)
    ap.add_argument("--sq-per-rank", type=int, default=32)
    ap.add_argument("--skv-per-rank", type=int, default=128)
    ap.add_argument("--tag", default="", help="suffix of the fixture's file name")
    ap.add_argument("--bias", action="store_true", help="run with the reference's bias_func protocol")
    a = ap.parse_args()
    import torch.multiprocessing as mp
    out = os.path.dirname(os.path.abspath(__file__))
    mp.spawn(worker, args=(a.world, a.ref, a.port, out, a.seed, a.heads, a.sq_per_rank, a.skv_per_rank, a.tag, a.bias),
             nprocs=a.world, join=True)
