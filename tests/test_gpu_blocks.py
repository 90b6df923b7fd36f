"""Several query blocks against one K/V shard in a single launch (the all-blocks-per-pass schedule), and the
two reduce kernels that finish it, through the C ABI wrappers, against the CPU oracle."""
import math

import pytest
import torch

import _parity
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128.0)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-4)])
def test_blocks_forward_backward(cuda_device, dtype, tol):
    from lv_xattn_b200 import ops, _lib
    n, B, Hq, Hkv, Sq, Skv = 3, 2, 4, 2, 96, 640
    d = cuda_device
    _, k, v, _ = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 50, dtype)
    valid = [640, 333]
    qs, dos, refs = [], [], []
    for i in range(n):
        q, _, _, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 51 + i, dtype)
        qs.append(q)
        dos.append(do)
        refs.append(orc.attention_fwd_bwd(q, k, v, do, SCALE, valid))
    q_all, do_all = torch.stack(qs).to(d), torch.stack(dos).to(d)
    kd, vd = k.to(d), v.to(d)
    kvl = torch.tensor(valid, dtype=torch.int32, device=d)
    o, lse = ops.fwd_block(q_all, kd, vd, SCALE, kv_valid_len=kvl)
    assert o.shape == q_all.shape and lse.shape == (n * B * Hq, Sq)
    delta = ops.bwd_prep(o, do_all)
    dq = torch.zeros(q_all.shape, dtype=torch.float32, device=d)
    dk = torch.full(k.shape, float("nan"), dtype=torch.float32, device=d)
    dv = torch.full(k.shape, float("nan"), dtype=torch.float32, device=d)
    ops.bwd_block(q_all, do_all, lse, delta, kd, vd, SCALE, dq, dk, dv, False, kv_valid_len=kvl)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    lse = lse.cpu().view(n, B, Hq, Sq)
    rel = 1e-2 if dtype != torch.float32 else 1e-4
    for i in range(n):
        o_ref, lse_ref, dq_ref, _, _ = refs[i]
        _parity.assert_close(o[i].float().cpu(), o_ref, "o", f"blocks{i}", tol, rel, 5 * rel)
        _parity.assert_lse_close(lse[i], lse_ref, f"blocks{i}", min(tol, 1e-3))
        _parity.assert_close(dq[i].cpu(), dq_ref, "dq", f"blocks{i}", tol, rel, 5 * rel)
    dk_ref = sum(r[3] for r in refs)
    dv_ref = sum(r[4] for r in refs)
    _parity.assert_close(dk.cpu(), dk_ref, "dk", "blocks", tol * 2, rel, 5 * rel)
    _parity.assert_close(dv.cpu(), dv_ref, "dv", "blocks", tol * 2, rel, 5 * rel)


def test_merge_parts_and_sum_cast(cuda_device):
    from lv_xattn_b200 import ops
    B, Hq, Hkv, Sq, Skv = 1, 4, 2, 64, 768
    d = cuda_device
    q, k, v, _ = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 60, torch.bfloat16)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, SCALE, [500])
    parts_o, parts_l = [], []
    for i, valid in enumerate([256, 244, 0]):            # three shards of 256 keys, the last one all padding
        kvl = torch.tensor([valid], dtype=torch.int32, device=d)
        o, l = ops.fwd_block(q.to(d), k[:, :, 256 * i:256 * (i + 1)].to(d), v[:, :, 256 * i:256 * (i + 1)].to(d), SCALE,
                             kv_valid_len=kvl, final=False)
        parts_o.append(o)
        parts_l.append(l)
    o, lse = ops.fwd_merge_parts(torch.stack(parts_o), torch.stack(parts_l), torch.bfloat16)
    _parity.assert_close(o.float().cpu(), o_ref, "o", "merge_parts", *_parity.BF16["o"])
    _parity.assert_lse_close(lse.cpu().view(B, Hq, Sq), lse_ref, "merge_parts")
    # all-empty merge stays (0, -inf)
    z = torch.zeros(2, 1, 1, 4, 128, device=d)
    ninf = torch.full((2, 1, 4), float("-inf"), device=d)
    o0, l0 = ops.fwd_merge_parts(z, ninf, torch.float32)
    assert torch.equal(o0.cpu(), torch.zeros(1, 1, 4, 128)) and torch.isinf(l0).all()
    parts = torch.randn(5, 3, 7, 128, device=d)
    s = ops.sum_cast(parts, torch.float32)
    assert torch.allclose(s, parts.sum(0), atol=1e-5)
    assert ops.sum_cast(parts, torch.bfloat16).dtype == torch.bfloat16


def test_gathered_blocks_with_in_kernel_waits(cuda_device):
    """lvx_fwd_block_gathered / lvx_bwd_block_gathered: the multi-block launch that starts with its own block and
    checks a per-block flag before touching the others. Here every flag is already at the epoch (the "peers" stored
    their blocks earlier in the same stream), so the kernels never wait for a later launch; results must equal the
    plain multi-block launch bit for bit (dQ: to fp32 reassociation), for every choice of the first block."""
    import ctypes
    from lv_xattn_b200 import ops, _lib
    n, B, Hq, Hkv, Sq, Skv = 4, 1, 8, 2, 128, 1024
    d = cuda_device
    _, k, v, _ = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 70, torch.bfloat16)
    qs = torch.stack([orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 71 + i, torch.bfloat16)[0] for i in range(n)]).to(d)
    dos = torch.stack([orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 71 + i, torch.bfloat16)[3] for i in range(n)]).to(d)
    kd, vd = k.to(d), v.to(d)
    o_ref, lse_ref = ops.fwd_block(qs, kd, vd, SCALE)
    delta = ops.bwd_prep(o_ref, dos)

    def bwd(block_wait):
        dq = torch.zeros(qs.shape, dtype=torch.float32, device=d)
        dk = torch.empty(k.shape, dtype=torch.bfloat16, device=d)
        dv = torch.empty(k.shape, dtype=torch.bfloat16, device=d)
        ops.bwd_block(qs, dos, lse_ref, delta, kd, vd, SCALE, dq, dk, dv, "final", block_wait=block_wait)
        return dq, dk, dv

    dq_ref, dk_ref, dv_ref = bwd(None)
    flags = torch.zeros(_lib.P2P_SLOTS * _lib.MAX_PEERS, dtype=torch.int32, device=d)
    flags.view(_lib.P2P_SLOTS, _lib.MAX_PEERS)[3, :n] = 7            # every block has reached epoch 7 on slot 3
    for first in range(n):
        for fl in (flags, None):                                      # with flags, and block order only
            part = ops.fwd_partials(qs, kd, vd, SCALE, block_wait=(fl, 3, 7, first))
            o = torch.empty_like(o_ref)
            lse = torch.empty_like(lse_ref)
            ops.fwd_combine(part, None, None, o, lse, True)
            assert torch.equal(o, o_ref) and torch.equal(lse, lse_ref)
            dq, dk, dv = bwd((fl, 3, 7, first))
            assert (dq - dq_ref).norm().item() <= 2e-5 * dq_ref.norm().item()
            # dK/dV sum over the blocks in TMEM in walk order: a different first block is a different fp32 order
            assert (dk.float() - dk_ref.float()).abs().max().item() <= 2e-2 * dk_ref.float().abs().max().item()
            assert (dv.float() - dv_ref.float()).abs().max().item() <= 2e-2 * dv_ref.float().abs().max().item()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    # a block whose flag nothing sets: with the limit at a millisecond the kernel gives up and says which block
    lib = _lib.load()
    try:
        _lib.check(lib.lvx_p2p_set_timeout(ctypes.c_double(1e-3)), "lvx_p2p_set_timeout")
        flags.view(_lib.P2P_SLOTS, _lib.MAX_PEERS)[3, 2] = 6          # block 2 is one epoch behind
        ops.fwd_partials(qs, kd, vd, SCALE, block_wait=(flags, 3, 7, 0))
        torch.cuda.synchronize()
        assert _lib.device_status() == (0x1300 | 2)
        bwd((flags, 3, 7, 1))
        torch.cuda.synchronize()
        assert _lib.device_status() == (0x1300 | 2)
    finally:
        _lib.check(lib.lvx_p2p_set_timeout(ctypes.c_double(120.0)), "lvx_p2p_set_timeout")
        _lib.device_status()
