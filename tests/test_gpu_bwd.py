"""Backward block through the C ABI against the CPU oracle's autograd backward (test.py:129-156 math).
Tolerance for 16-bit inputs: dQ/dK/dV max-abs <= 2e-2 against the fp32 oracle on the same rounded inputs, plus
the relative criteria of tests/_parity.py (an all-zero or mis-scaled gradient fails at any sequence length)."""
import math

import pytest
import torch

import _parity
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


def check(got, ref, label="bwd"):
    _parity.assert_grads_16bit(got, ref, label)


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
    check(*run_case(cuda_device, *shape, dtype), label=f"bwd{shape}{dtype}")


@pytest.mark.parametrize("skv", [32, 100, 129, 1000])
def test_bwd_ragged_kv(cuda_device, skv):
    check(*run_case(cuda_device, 1, 4, 2, 96, skv, torch.bfloat16, seed=3), label=f"bwd_ragged{skv}")


def test_bwd_key_padding(cuda_device):
    check(*run_case(cuda_device, 3, 4, 2, 128, 1024, torch.bfloat16, seed=5, kv_valid=[1024, 300, 0]), label="bwd_keypad")


def test_bwd_accumulate_over_steps(cuda_device):
    check(*run_case(cuda_device, 1, 8, 2, 256, 1024, torch.bfloat16, seed=9, two_steps=True), label="bwd_two_steps")


@pytest.mark.parametrize("case", [
    (1, 1, 1, 64, 128 * 300, None),                 # one query tile per K/V tile: every barrier phase flips per item
    (2, 2, 2, 320, 128 * 120, [128 * 120, 7000]),   # three query tiles per item; 65 tiles of batch entry 1 hold no valid key
    (1, 4, 2, 96, 128 * 200 + 37, None),            # ragged last K/V tile at the end of a CTA's walk
])
@pytest.mark.parametrize("final_dtype", [False, True])
def test_bwd_many_items_per_cta(cuda_device, case, final_dtype):
    """The grid is persistent (one CTA per SM), so with more K/V tiles than SMs a CTA walks several of them back to
    back, some of them without any valid key. dK/dV in fp32 and written directly in the input dtype."""
    from lv_xattn_b200 import ops, _lib
    B, Hq, Hkv, Sq, Skv, valid = case
    if not final_dtype:
        check(*run_case(cuda_device, B, Hq, Hkv, Sq, Skv, torch.bfloat16, seed=13, kv_valid=valid), label=f"bwd_items{case}")
        return
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 13, torch.bfloat16)
    ref = orc.attention_fwd_bwd(q, k, v, do, SCALE, valid)
    d = cuda_device
    qd, kd, vd, dod = q.to(d), k.to(d), v.to(d), do.to(d)
    kvl = None if valid is None else torch.tensor(valid, dtype=torch.int32, device=d)
    o, lse = ops.fwd_block(qd, kd, vd, SCALE, kv_valid_len=kvl)
    delta = ops.bwd_prep(o, dod)
    dq = torch.zeros(B, Hq, Sq, 128, dtype=torch.float32, device=d)
    dk = torch.full((B, Hkv, Skv, 128), float("nan"), dtype=torch.bfloat16, device=d)
    dv = torch.full((B, Hkv, Skv, 128), float("nan"), dtype=torch.bfloat16, device=d)
    ops.bwd_block(qd, dod, lse, delta, kd, vd, SCALE, dq, dk, dv, "final", kvl)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    check((dq.cpu(), dk.float().cpu(), dv.float().cpu()), ref[2:], label=f"bwd_items_final{case}")


def test_bwd_run_twice(cuda_device):
    """dK/dV are accumulated in TMEM by one CTA per K/V tile in a fixed order: two runs agree bit for bit. dQ is
    reduce-added in fp32 by all K/V tiles in whatever order they finish, so two runs differ by fp32
    reassociation only: relative Frobenius difference <= 2e-5 (64 partials per element here)."""
    from lv_xattn_b200 import ops
    B, Hq, Hkv, Sq, Skv = 1, 8, 2, 512, 8192
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 77, torch.bfloat16)
    d = cuda_device
    qd, kd, vd, dod = q.to(d), k.to(d), v.to(d), do.to(d)
    o, lse = ops.fwd_block(qd, kd, vd, SCALE)
    delta = ops.bwd_prep(o, dod)
    runs = []
    for _ in range(2):
        dq = torch.zeros(B, Hq, Sq, 128, dtype=torch.float32, device=d)
        dk = torch.empty(B, Hkv, Skv, 128, dtype=torch.float32, device=d)
        dv = torch.empty(B, Hkv, Skv, 128, dtype=torch.float32, device=d)
        ops.bwd_block(qd, dod, lse, delta, kd, vd, SCALE, dq, dk, dv, False)
        runs.append((dq, dk, dv))
    torch.cuda.synchronize()
    assert torch.equal(runs[0][1], runs[1][1]) and torch.equal(runs[0][2], runs[1][2])
    diff = (runs[0][0] - runs[1][0]).norm().item() / runs[0][0].norm().item()
    assert diff <= 2e-5, diff
