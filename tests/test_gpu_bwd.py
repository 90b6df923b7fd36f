"""Backward block through the C ABI against the CPU oracle's autograd backward (test.py:129-156 math).
Tolerance for 16-bit inputs: dQ/dK/dV max-abs <= 2e-2 against the fp32 oracle on the same rounded inputs."""
import math

import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128.0)


def run_case(device, B, Hq, Hkv, Sq, Skv, dtype, seed=1, kv_valid=None, two_steps=False):
    from lv_xattn_b200 import ops, _lib
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, seed, dtype)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = orc.attention_fwd_bwd(q, k, v, do, SCALE, kv_valid)
    d = device
    qd, kd, vd, dod = q.to(d), k.to(d), v.to(d), do.to(d)
    kvl = None if kv_valid is None else torch.tensor(kv_valid, dtype=torch.int32, device=d)
    o, lse = ops.fwd_block(qd, kd, vd, SCALE, kv_valid_len=kvl)
    delta = ops.bwd_prep(o, dod)
    dq = torch.zeros(B, Hq, Sq, 128, dtype=torch.float32, device=d)
    dk = torch.full((B, Hkv, Skv, 128), float("nan"), dtype=torch.float32, device=d)
    dv = torch.full((B, Hkv, Skv, 128), float("nan"), dtype=torch.float32, device=d)
    if not two_steps:
        ops.bwd_block(qd, dod, lse, delta, kd, vd, SCALE, dq, dk, dv, False, kv_valid_len=kvl)
    else:
        # the query block split in two halves, second call accumulating into dk/dv (the step-loop pattern)
        h = Sq // 2
        lse3, delta3 = lse.view(B, Hq, Sq), delta.view(B, Hq, Sq)
        for i, (a, b) in enumerate(((0, h), (h, Sq))):
            dq_part = torch.zeros(B, Hq, b - a, 128, dtype=torch.float32, device=d)
            ops.bwd_block(qd[:, :, a:b].contiguous(), dod[:, :, a:b].contiguous(),
                          lse3[:, :, a:b].contiguous().view(B * Hq, b - a),
                          delta3[:, :, a:b].contiguous().view(B * Hq, b - a), kd, vd, SCALE, dq_part, dk, dv, i > 0,
                          kv_valid_len=kvl)
            dq[:, :, a:b] = dq_part
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return (dq.cpu(), dk.cpu(), dv.cpu()), (dq_ref, dk_ref, dv_ref)


def check(got, ref, tol=2e-2):
    for name, g, r in zip(("dQ", "dK", "dV"), got, ref):
        assert not torch.isnan(g).any(), f"{name} has NaN"
        err = (g - r).abs().max().item()
        assert err <= tol, f"{name} max-abs err {err} (ref max {r.abs().max().item()})"


@pytest.mark.parametrize("shape", [
    (1, 1, 1, 64, 128),
    (1, 1, 1, 128, 128),
    (1, 2, 1, 128, 256),
    (1, 4, 1, 80, 1024),       # ragged packed rows (320 = 5 tiles of 64)
    (2, 8, 2, 192, 2048),
    (1, 32, 8, 512, 8192),     # the reference's correctness shape, 16-bit inputs
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_bwd_shapes(cuda_device, shape, dtype):
    check(*run_case(cuda_device, *shape, dtype))


@pytest.mark.parametrize("skv", [32, 100, 129, 1000])
def test_bwd_ragged_kv(cuda_device, skv):
    check(*run_case(cuda_device, 1, 4, 2, 96, skv, torch.bfloat16, seed=3))


def test_bwd_key_padding(cuda_device):
    check(*run_case(cuda_device, 3, 4, 2, 128, 1024, torch.bfloat16, seed=5, kv_valid=[1024, 300, 0]))


def test_bwd_accumulate_over_steps(cuda_device):
    check(*run_case(cuda_device, 1, 8, 2, 256, 1024, torch.bfloat16, seed=9, two_steps=True))
