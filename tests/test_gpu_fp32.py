"""fp32 inputs (the reference's CPU-runnable correctness configuration): |err| <= 1e-4 on O, lse, dQ, dK, dV
against the fp32 CPU oracle, through the Python entry points."""
import math

import pytest
import torch

import _parity
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128.0)


def run(device, B, Hq, Hkv, Sq, Skv, seed, kv_valid=None):
    import lv_xattn_b200 as lvx
    from lv_xattn_b200 import _lib
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, seed, torch.float32)
    ref = orc.attention_fwd_bwd(q, k, v, do, SCALE, kv_valid)
    qd, kd, vd, dod = (t.to(device) for t in (q, k, v, do))
    _, _, _, o, L = lvx._attn_forward(qd, kd, vd, False, SCALE, None, kv_valid_len=kv_valid)
    dq, dk, dv = lvx._attn_backward(dod, qd, kd, vd, o, L, False, SCALE, None, "flash", kv_valid_len=kv_valid)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert o.dtype == torch.float32 and dq.dtype == torch.float32
    got = (o.cpu(), L.cpu().view(B, Hq, Sq), dq.cpu(), dk.cpu(), dv.cpu())
    return got, ref


def check(got, ref, tol=1e-4):
    _parity.assert_lse_close(got[1], ref[1], "fp32", tol)
    for name, g, r in zip(("o", "lse", "dq", "dk", "dv"), got, ref):
        if name != "lse":
            _parity.assert_fp32(g, r, name, "fp32")


def test_config1_shape(cuda_device):
    # B=1, 32 query heads, 8 KV heads, 512 queries, 8192 keys, fp32, no mask, scale 1/sqrt(128)
    check(*run(cuda_device, 1, 32, 8, 512, 8192, 1))


@pytest.mark.parametrize("shape", [(1, 1, 1, 64, 64), (2, 4, 2, 40, 200), (1, 8, 2, 96, 1000)])
def test_small_and_ragged(cuda_device, shape):
    check(*run(cuda_device, *shape, 2))


def test_key_padding(cuda_device):
    check(*run(cuda_device, 3, 4, 2, 64, 512, 3, kv_valid=[512, 130, 0]))
