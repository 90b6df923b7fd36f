"""The general block kernels with a dense additive bias (the reference's bias_func protocol, lv_xattn/attn.py:386-389:
S = sm_scale*q.k + bias) through the C ABI, for every input dtype, against the CPU oracle. 16-bit tolerances as in the
other tests (2e-2 max-abs, lse 1e-3, plus the relative criteria); fp32 1e-4."""
import math

import pytest
import torch

import _parity
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128.0)


def make_bias(B, Hb, Sq, Skv, seed, mask_every=0):
    g = torch.Generator().manual_seed(seed)
    bias = torch.randn(B, Hb, Sq, Skv, generator=g)
    if mask_every:
        bias[..., ::mask_every] = float("-inf")
    return bias


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [
    (1, 2, 1, 64, 128, 1),       # one 64x64 tile pair, bias broadcast over heads
    (2, 4, 2, 80, 300, 4),       # ragged rows and keys, per-head bias, GQA
    (1, 8, 2, 256, 2048, 1),
])
def test_bias_forward_backward(cuda_device, shape, dtype):
    from lv_xattn_b200 import ops, _lib
    B, Hq, Hkv, Sq, Skv, Hb = shape
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 61, dtype)
    bias = make_bias(B, Hb, Sq, Skv, 62, mask_every=5)
    ref = orc.attention_fwd_bwd(q, k, v, do, SCALE, bias=bias)
    d = cuda_device
    qd, kd, vd, dod, bd = (t.to(d) for t in (q, k, v, do, bias))
    o, lse = ops.fwd_block(qd, kd, vd, SCALE, bias=bd)
    delta = ops.bwd_prep(o, dod)
    dq = torch.zeros(B, Hq, Sq, 128, dtype=torch.float32, device=d)
    dk = torch.empty(B, Hkv, Skv, 128, dtype=torch.float32, device=d)
    dv = torch.empty(B, Hkv, Skv, 128, dtype=torch.float32, device=d)
    ops.bwd_block(qd, dod, lse, delta, kd, vd, SCALE, dq, dk, dv, False, bias=bd)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    label = f"bias{shape}{dtype}"
    got = (o.float().cpu(), lse.cpu().view(B, Hq, Sq), dq.cpu(), dk.cpu(), dv.cpu())
    if dtype == torch.float32:
        _parity.assert_lse_close(got[1], ref[1], label, 1e-4)
        for name, g_, r in zip(("o", "dq", "dk", "dv"), (got[0],) + got[2:], (ref[0],) + ref[2:]):
            _parity.assert_fp32(g_, r, name, label)
    else:
        _parity.assert_lse_close(got[1], ref[1], label)
        _parity.assert_close(got[0], ref[0], "o", label, *_parity.BF16["o"])
        _parity.assert_grads_16bit(got[2:], ref[2:], label)


def test_bias_through_the_entry_points_with_key_padding(cuda_device):
    """_attn_forward/_attn_backward with bias_func(*local, *remote) and kv_valid_len together; dK/dV come back in the
    input dtype (accumulate mode 2 of the general kernels)."""
    import lv_xattn_b200 as lvx
    B, Hq, Hkv, Sq, Skv = 2, 4, 2, 96, 640
    valid = [640, 333]
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 63, torch.bfloat16)
    key_term, qry_term = torch.randn(Skv), torch.randn(Sq)
    bias = (qry_term[:, None] + key_term[None, :])[None, None].expand(B, 1, Sq, Skv).contiguous()
    ref = orc.attention_fwd_bwd(q, k, v, do, SCALE, valid, bias=bias)
    d = cuda_device
    kw = dict(bias_func=lambda ka, qa: (qa[:, None] + ka[None, :])[None, None],
              local_bias_args=[key_term.to(d)], remote_bias_args=[qry_term.to(d)], kv_valid_len=valid)
    qd, kd, vd, dod = (t.to(d) for t in (q, k, v, do))
    _, _, _, o, L = lvx._attn_forward(qd, kd, vd, False, SCALE, None, **kw)
    dq, dk, dv = lvx._attn_backward(dod, qd, kd, vd, o, L, False, SCALE, None, "flash", **kw)
    assert dk.dtype == torch.bfloat16
    _parity.assert_lse_close(L.cpu().view(B, Hq, Sq), ref[1], "bias_api")
    _parity.assert_close(o.float().cpu(), ref[0], "o", "bias_api", *_parity.BF16["o"])
    _parity.assert_grads_16bit((dq, dk, dv), ref[2:], "bias_api")
