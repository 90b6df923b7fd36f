"""The reference-facing Python entry points on one GPU: _attn_forward / _attn_backward, the save-QKV autograd
wrapper and the recompute-QKV wrapper, against the CPU oracle."""
import math

import pytest
import torch

import _parity
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128.0)


def test_forward_backward_entry_points(cuda_device):
    import lv_xattn_b200 as lvx
    B, Hq, Hkv, Sq, Skv = 2, 8, 2, 128, 1024
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 21, torch.bfloat16)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = orc.attention_fwd_bwd(q, k, v, do, SCALE, [1024, 700])
    d = cuda_device
    qd, kd, vd, dod = (t.to(d) for t in (q, k, v, do))
    q2, k2, v2, o, L = lvx._attn_forward(qd, kd, vd, False, SCALE, None, kv_valid_len=[1024, 700])
    assert q2 is qd and k2 is kd and v2 is vd
    assert o.shape == qd.shape and o.dtype == qd.dtype and L.shape == (B * Hq, Sq) and L.dtype == torch.float32
    dq, dk, dv = lvx._attn_backward(dod, qd, kd, vd, o, L, False, SCALE, None, "flash", kv_valid_len=[1024, 700])
    assert dq.shape == qd.shape and dk.shape == kd.shape and dv.shape == vd.shape and dk.dtype == kd.dtype
    _parity.assert_close(o.float().cpu(), o_ref, "o", "api_entry", *_parity.BF16["o"])
    _parity.assert_lse_close(L.cpu().view(B, Hq, Sq), lse_ref, "api_entry")
    _parity.assert_grads_16bit((dq, dk, dv), (dq_ref, dk_ref, dv_ref), "api_entry")


def test_autograd_wrapper(cuda_device):
    import lv_xattn_b200 as lvx
    B, Hq, Hkv, Sq, Skv = 1, 4, 4, 256, 512
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 22, torch.float16)
    _, _, dq_ref, dk_ref, dv_ref = orc.attention_fwd_bwd(q, k, v, do, SCALE)
    d = cuda_device
    qd, kd, vd = (t.to(d).requires_grad_(True) for t in (q, k, v))
    attention = lvx.create_attention_class("lv_xattn").apply
    o = attention(qd, kd, vd, False, SCALE)
    o.backward(do.to(d))
    _parity.assert_grads_16bit((qd.grad, kd.grad, vd.grad), (dq_ref, dk_ref, dv_ref), "api_autograd")


def test_recompute_wrapper_propagates_gradients(cuda_device):
    """K/V are recomputed in backward and the gradients reach x and the projection weights (the reference's
    wrapper drops them, test_llama3.py:243)."""
    import lv_xattn_b200 as lvx
    d = cuda_device
    torch.manual_seed(3)
    B, Sq, Skv, H, hid = 1, 64, 512, 2, 256
    x = (torch.randn(B, Sq, hid, device=d) * 0.5).bfloat16().requires_grad_(True)
    states = (torch.randn(B, Skv, hid, device=d) * 0.5).bfloat16()
    wq, wk, wv = ((torch.randn(hid, H * 128, device=d) * 0.05).bfloat16().requires_grad_(True) for _ in range(3))

    def project(xx, st):
        q = (xx @ wq).view(B, Sq, H, 128).transpose(1, 2)
        k = (st @ wk).view(B, Skv, H, 128).transpose(1, 2)
        v = (st @ wv).view(B, Skv, H, 128).transpose(1, 2)
        return q, k, v

    o = lvx.LVXAttnRecomputeFunc.apply(x, project, False, lambda: states, None, wq, wk, wv)
    go = torch.randn_like(o)
    o.backward(go)
    got = [t.grad.float().clone() for t in (x, wq, wk, wv)]
    for t in (x, wq, wk, wv):
        t.grad = None
    # same layer with plain fp32 attention math through autograd
    q, k, v = project(x, states)
    p = torch.softmax((q.float() @ k.float().transpose(2, 3)) * (128 ** -0.5), dim=-1)
    o_ref = (p @ v.float())
    o_ref.backward(go.float())
    assert (o.float() - o_ref).abs().max() <= 2e-2
    for g, t in zip(got, (x, wq, wk, wv)):
        ref = t.grad.float()
        assert (g - ref).abs().max() <= 3e-2 * max(1.0, ref.abs().max().item()), (g - ref).abs().max()


def _golden_files():
    import glob
    import os
    return sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "ref_lvxattn_w*.npz")))


@pytest.mark.parametrize("path", _golden_files(), ids=lambda p: p.rsplit("/", 1)[-1])
def test_against_reference_golden_vectors(cuda_device, path):
    """The CUDA path on the inputs of tests/golden/*.npz against what the reference's own implementation produced
    for them (fp16; W = 1, 2, 4 -- the full tensors are run on one GPU and compared shard by shard).

    The reference's +1 in the softmax denominator (lv_xattn/attn.py:319) equals one extra key with score 0 and
    value 0, so the kernels are given [K; 0], [V; 0] (a ragged 128*W + 1 keys) and must then reproduce the
    reference's O, L, dQ, dK, dV to fp16 rounding: relative Frobenius error <= 2e-3, lse <= 1e-4."""
    import numpy as np
    import lv_xattn_b200 as lvx
    g = np.load(path)
    W = int(g["world"])
    q, k, v, do = (torch.from_numpy(g[n]).to(cuda_device) for n in ("q", "k", "v", "do"))
    zero = torch.zeros_like(k[:, :, :1])
    ke, ve = torch.cat([k, zero], 2).contiguous(), torch.cat([v, zero], 2).contiguous()
    scale = float(g["scale"])
    kw = {}
    if "bias" in g.files:       # fixture made with the reference's bias_func protocol: the general (bias) kernels
        bias = torch.from_numpy(g["bias"]).to(cuda_device)
        bias = torch.cat([bias, torch.zeros_like(bias[..., :1])], -1).contiguous()
        kw = dict(bias_func=lambda b: b, local_bias_args=[bias], remote_bias_args=[])
    _, _, _, o, L = lvx._attn_forward(q, ke, ve, False, scale, None, **kw)
    dq, dk, dv = lvx._attn_backward(do, q, ke, ve, o, L, False, scale, None, "flash", **kw)
    B, H, Sq, D = q.shape
    got = {"o": o.float().cpu(), "dq": dq.float().cpu(), "dk": dk[:, :, :-1].float().cpu(), "dv": dv[:, :, :-1].float().cpu()}
    L = L.cpu().view(B, H, Sq)
    for r in range(W):
        L_ref = torch.from_numpy(g["ref_L"][r]).view(B, H, Sq // W)
        assert (orc.shard(L.unsqueeze(-1), r, W).squeeze(-1) - L_ref).abs().max() <= 1e-4
        for name, full in got.items():
            ref = torch.from_numpy(g[f"ref_{name}"][r].astype(np.float32))
            _parity.assert_close(orc.shard(full, r, W), ref, name, f"golden_w{W}_r{r}", 1e-2, 2e-3, 5e-3)


@pytest.mark.parametrize("chunks,valid", [(1, None), (3, None), (4, [700, 1000])])
def test_host_streamed_attention(cuda_device, chunks, valid):
    """Pinned host tensors in and out, K/V streamed in chunks: same results as the oracle."""
    import lv_xattn_b200 as lvx
    B, Hq, Hkv, Sq, Skv = 2, 8, 2, 128, 1000
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 23, torch.bfloat16)
    ref = orc.attention_fwd_bwd(q, k, v, do, SCALE, valid)
    hq, hk, hv, hdo = (t.pin_memory() for t in (q, k, v, do))
    ho, hdq = torch.empty_like(hq).pin_memory(), torch.empty_like(hq).pin_memory()
    hdk, hdv = torch.empty_like(hk).pin_memory(), torch.empty_like(hk).pin_memory()
    st = lvx.HostStreamedAttention(cuda_device, chunks=chunks)
    for _ in range(2):      # twice: device buffers and streams are reused
        st.step(hq, hk, hv, hdo, SCALE, ho, hdq, hdk, hdv, kv_valid_len=valid)
    for name, got, r in zip(("o", "dq", "dk", "dv"), (ho, hdq, hdk, hdv), (ref[0], ref[2], ref[3], ref[4])):
        _parity.assert_close(got.float(), r, name, f"host_streamed_{chunks}", *_parity.BF16[name])


def test_host_streamed_attention_pipelined(cuda_device):
    """Three steps with DIFFERENT inputs, each prefetched while the one before is queued and none waited for until
    the end: every step's results (its own host output tensors) match the oracle, so neither an input set nor an
    output buffer was reused too early."""
    import lv_xattn_b200 as lvx
    B, Hq, Hkv, Sq, Skv = 1, 8, 2, 128, 1000
    st = lvx.HostStreamedAttention(cuda_device, chunks=3)
    steps = []
    for seed in (31, 32, 33):
        q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, seed, torch.bfloat16)
        host = [t.pin_memory() for t in (q, k, v, do)]
        outs = [torch.empty_like(host[0]).pin_memory(), torch.empty_like(host[0]).pin_memory(),
                torch.empty_like(host[1]).pin_memory(), torch.empty_like(host[1]).pin_memory()]
        steps.append((host, outs, orc.attention_fwd_bwd(q, k, v, do, SCALE, None)))
    st.prefetch(*steps[0][0])
    for i, (host, outs, _) in enumerate(steps):
        if i + 1 < len(steps):
            st.prefetch(*steps[i + 1][0])
        st.step(*host, SCALE, *outs, wait=False)
    with pytest.raises(RuntimeError):          # two sets at most
        st.prefetch(*steps[0][0])
        st.prefetch(*steps[1][0])
        st.prefetch(*steps[2][0])
    st.finish()
    for i, (_, outs, ref) in enumerate(steps):
        for name, got, r in zip(("o", "dq", "dk", "dv"), outs, (ref[0], ref[2], ref[3], ref[4])):
            _parity.assert_close(got.float(), r, name, f"host_pipelined_step{i}", *_parity.BF16[name])
