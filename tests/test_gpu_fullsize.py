"""The benchmark's full single-GPU sizes, where the CPU oracle is out of reach.

Checked against the oracle's per-KV-group fp32 form run on the GPU (oracle.group_fwd_bwd: plain fp32 torch
matmuls, one head at a time -- the torch fp32 reference of the same op): for two KV groups of each shape EVERY
row of O, lse and dQ of their query heads and EVERY key of dK and dV, under the absolute bars (2e-2, lse 1e-3)
and the relative ones of tests/_parity.py (at these lengths |O| ~ 7e-3, so only the relative bars can fail).
Plus size-independent properties:
  * V = 1 everywhere  =>  O = 1 exactly (softmax rows sum to one) and dK = dQ = 0 up to rounding
  * attention over the whole K/V == merge of attention over its two halves (the shard merge identity)
  * the backward is linear in dO:  grad(2*dO) = 2*grad(dO)
"""
import math

import pytest
import torch

import _parity
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128.0)
B, HQ, HKV, SQ, SKV = 1, 32, 8, 2048, 131072
G = HQ // HKV


@pytest.fixture(scope="module")
def tensors(cuda_device):
    g = torch.Generator(device=cuda_device).manual_seed(7)
    q = torch.empty(B, HQ, SQ, 128, device=cuda_device).normal_(0, 0.5, generator=g).bfloat16()
    k = torch.empty(B, HKV, SKV, 128, device=cuda_device).normal_(0, 0.5, generator=g).bfloat16()
    v = torch.empty(B, HKV, SKV, 128, device=cuda_device).normal_(0, 0.5, generator=g).bfloat16()
    do = torch.empty(B, HQ, SQ, 128, device=cuda_device).normal_(0, 1.0, generator=g).bfloat16()
    return q, k, v, do


def check_groups(label, groups, q, k, v, do, o, L, dq, dk, dv, valid=None):
    """groups: (batch, kv head) pairs; everything those groups produce against the fp32 group reference."""
    Bz, Hq, Sq, _ = q.shape
    L3 = L.view(Bz, Hq, Sq)
    for b, hk in groups:
        hs = slice(hk * G, (hk + 1) * G)
        n = None if valid is None else valid[b]
        o_r, lse_r, dq_r, dk_r, dv_r = orc.group_fwd_bwd(q[b, hs], k[b, hk], v[b, hk], do[b, hs], SCALE, n)
        tag = f"{label}_b{b}_kv{hk}"
        _parity.assert_lse_close(L3[b, hs], lse_r, tag)
        _parity.assert_close(o[b, hs].float(), o_r, "o", tag, *_parity.BF16["o"])
        _parity.assert_close(dq[b, hs].float(), dq_r, "dq", tag, *_parity.BF16["dq"])
        _parity.assert_close(dk[b, hk].float(), dk_r, "dk", tag, *_parity.BF16["dk"])
        _parity.assert_close(dv[b, hk].float(), dv_r, "dv", tag, *_parity.BF16["dv"])


def test_benchmark_shape_against_fp32_reference(tensors):
    """B=1, Hq=32, Hkv=8, Sq=2048, Skv=131072, bf16: KV groups 0 and 5 in full."""
    import lv_xattn_b200 as lvx
    from lv_xattn_b200 import _lib
    q, k, v, do = tensors
    _, _, _, o, L = lvx._attn_forward(q, k, v, False, SCALE, None)
    dq, dk, dv = lvx._attn_backward(do, q, k, v, o, L, False, SCALE, None, "flash")
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    check_groups("config2", [(0, 0), (0, 5)], q, k, v, do, o, L, dq, dk, dv)


def test_constant_v_gives_constant_o(tensors):
    import lv_xattn_b200 as lvx
    q, k, v, do = tensors
    ones = torch.ones_like(v)
    _, _, _, o, L = lvx._attn_forward(q, k, ones, False, SCALE, None)
    assert torch.equal(o, torch.ones_like(o))
    dq, dk, dv = lvx._attn_backward(do, q, k, ones, o, L, False, SCALE, None, "flash")
    # dP = dO V^T is constant along keys and equals delta = rowsum(dO), so dS = P*(dP - delta) vanishes up to the
    # summation order of the two row sums: ~1e-5 * P, far below the ~1e-3 these gradients have for random V
    assert dq.float().abs().max().item() <= 1e-5
    assert dk.float().abs().max().item() <= 1e-5
    # dV[j] = sum_i P[i,j] dO[i]: finite and not identically zero
    assert torch.isfinite(dv.float()).all() and dv.float().abs().max().item() > 0


def test_merge_of_halves_equals_whole(tensors):
    from lv_xattn_b200 import ops
    q, k, v, _ = tensors
    h = SKV // 2
    o_full, l_full = ops.fwd_block(q, k, v, SCALE)
    o1, l1 = ops.fwd_block(q, k[:, :, :h].contiguous(), v[:, :, :h].contiguous(), SCALE, final=False)
    o2, l2 = ops.fwd_block(q, k[:, :, h:].contiguous(), v[:, :, h:].contiguous(), SCALE, o_in=o1, lse_in=l1)
    # both sides are rounded to bf16 once: relative Frobenius distance of two roundings of the same value ~1.6e-3
    _parity.assert_close(o2.float(), o_full.float(), "o", "merge_halves", 4e-3, 5e-3, 2e-2)
    assert (l_full - l2).abs().max().item() <= 1e-4


def test_backward_is_linear_in_do(tensors):
    import lv_xattn_b200 as lvx
    q, k, v, do = tensors
    _, _, _, o, L = lvx._attn_forward(q, k, v, False, SCALE, None)
    g1 = lvx._attn_backward(do, q, k, v, o, L, False, SCALE, None, "flash")
    g2 = lvx._attn_backward((do.float() * 2).bfloat16(), q, k, v, o, L, False, SCALE, None, "flash")
    for name, a, b in zip(("dq", "dk", "dv"), g1, g2):   # scaling by 2 is exact in bf16: only the final roundings differ
        _parity.assert_close(a.float() * 2, b.float(), name, "linear_in_do", 1e-2, 5e-3, 2e-2)


def test_long_visual_stress_shape_with_key_padding(cuda_device):
    """The long-visual stress shape on one GPU: B=2, Sq=256, 1,048,576 keys per sample, valid lengths
    1,048,576 and 786,432. KV groups (0, 0) and (1, 7) in full against the fp32 group reference; gradients of
    padded keys are exactly zero."""
    import lv_xattn_b200 as lvx
    from lv_xattn_b200 import _lib
    d = cuda_device
    Bz, Sq, Skv = 2, 256, 1048576
    valid = [1048576, 786432]
    g = torch.Generator(device=d).manual_seed(11)
    q = torch.empty(Bz, HQ, Sq, 128, device=d).normal_(0, 0.5, generator=g).bfloat16()
    k = torch.empty(Bz, HKV, Skv, 128, device=d).normal_(0, 0.5, generator=g).bfloat16()
    v = torch.empty(Bz, HKV, Skv, 128, device=d).normal_(0, 0.5, generator=g).bfloat16()
    do = torch.empty(Bz, HQ, Sq, 128, device=d).normal_(0, 1.0, generator=g).bfloat16()
    _, _, _, o, L = lvx._attn_forward(q, k, v, False, SCALE, None, kv_valid_len=valid)
    dq, dk, dv = lvx._attn_backward(do, q, k, v, o, L, False, SCALE, None, "flash", kv_valid_len=valid)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.isfinite(o.float()).all() and torch.isfinite(dq.float()).all()
    assert dk[1, :, valid[1]:].abs().max().item() == 0.0 and dv[1, :, valid[1]:].abs().max().item() == 0.0
    assert dk[1, :, :valid[1]].abs().max().item() > 0.0
    check_groups("config5", [(0, 0), (1, 7)], q, k, v, do, o, L, dq, dk, dv, valid)
