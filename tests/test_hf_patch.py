"""The Hugging Face hooks on the installed transformers' Mllama text attention modules, against the stock
modules with the same weights. On CPU the flash kernels are replaced by the tests-only torch stub, so this
checks the hook plumbing: projections, per-head RMSNorm, native GQA, K/V recompute and gradient flow into the
hidden states and every weight. (The GPU variant with the real kernels is tests/test_gpu_hf_patch.py.)"""
import copy

import pytest
import torch

mllama = pytest.importorskip("transformers.models.mllama.modeling_mllama")


def make_modules(hidden=256, heads=2, kv_heads=1, dtype=torch.float32):
    cfg = mllama.MllamaTextConfig(hidden_size=hidden, num_attention_heads=heads, num_key_value_heads=kv_heads,
                                  num_hidden_layers=2, intermediate_size=512, vocab_size=64)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    cross = mllama.MllamaTextCrossAttention(cfg, layer_idx=0).to(dtype)
    selfa = mllama.MllamaTextSelfAttention(cfg, layer_idx=1).to(dtype)
    rope = mllama.MllamaRotaryEmbedding(cfg)
    return cfg, cross, selfa, rope


def test_cross_attention_hook_matches_stock_module(monkeypatch):
    import _stub_ops
    import lv_xattn_b200.attn as attn
    from lv_xattn_b200 import hf_patch
    monkeypatch.setattr(attn, "ops", _stub_ops)
    cfg, cross, _, _ = make_modules()
    patched = copy.deepcopy(cross)
    patched.forward = hf_patch.patch_cross_attention_forward("lv_xattn").__get__(patched)
    x = torch.randn(2, 24, 256, requires_grad=True)
    states = torch.randn(2, 80, 256)
    ref, _ = cross(x, cross_attention_states=states)
    g = torch.randn_like(ref)
    ref.backward(g)
    ref_grads = [x.grad.clone()] + [p.grad.clone() for p in cross.parameters()]
    x.grad = None
    hf_patch.set_global_cross_attention_states(states)
    try:
        out, w = patched(x)
        assert w is None
        out.backward(g)
    finally:
        hf_patch.clear_global_cross_attention_states()
    assert torch.allclose(out, ref, atol=2e-5, rtol=1e-4)
    got = [x.grad] + [p.grad for p in patched.parameters()]
    for a, b, name in zip(got, ref_grads, ["x"] + [n for n, _ in cross.named_parameters()]):
        assert a is not None, name
        assert torch.allclose(a, b, atol=5e-5, rtol=1e-3), (name, (a - b).abs().max())


def test_cross_attention_hook_uses_the_states_of_each_call(monkeypatch):
    """Two forwards with different visual states passed as arguments (the normal Hugging Face call path), both
    before any backward: each output and each backward must belong to its own states."""
    import _stub_ops
    import lv_xattn_b200.attn as attn
    from lv_xattn_b200 import hf_patch
    monkeypatch.setattr(attn, "ops", _stub_ops)
    cfg, cross, _, _ = make_modules()
    patched = copy.deepcopy(cross)
    patched.forward = hf_patch.patch_cross_attention_forward("lv_xattn").__get__(patched)
    hf_patch.clear_global_cross_attention_states()
    x = torch.randn(1, 12, 256)
    st_a, st_b = torch.randn(1, 40, 256), torch.randn(1, 56, 256)
    try:
        xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        out_a, _ = patched(xa, cross_attention_states=st_a)
        out_b, _ = patched(xb, cross_attention_states=st_b)          # second batch: new states
        g = torch.randn_like(out_a)
        out_a.backward(g)                                            # recompute must still see st_a
        out_b.backward(g)
    finally:
        hf_patch.clear_global_cross_attention_states()
    for st, out, xg in ((st_a, out_a, xa.grad), (st_b, out_b, xb.grad)):
        xr = x.clone().requires_grad_(True)
        ref, _ = cross(xr, cross_attention_states=st)
        ref.backward(g)
        assert torch.allclose(out, ref, atol=2e-5, rtol=1e-4)
        assert torch.allclose(xg, xr.grad, atol=5e-5, rtol=1e-3)
    assert not torch.allclose(out_a, out_b, atol=1e-3)


def test_self_attention_hook_matches_stock_module_single_rank():
    from lv_xattn_b200 import hf_patch
    cfg, _, selfa, rope = make_modules()
    patched = copy.deepcopy(selfa)
    patched.forward = hf_patch.patch_self_attention_forward("lv_xattn").__get__(patched)
    x = torch.randn(2, 16, 256)
    pos = torch.arange(16)[None].expand(2, -1)
    pe = rope(x, pos)
    causal = torch.full((16, 16), float("-inf")).triu(1)[None, None].expand(2, 1, -1, -1)
    ref, _ = selfa(x, attention_mask=causal, position_embeddings=pe)
    out, _ = patched(x, attention_mask=None, position_embeddings=pe)
    assert torch.allclose(out, ref, atol=2e-5, rtol=1e-4)


def test_attention_modes():
    """The reference's three modes are accepted (test_llama3.py:107); anything else raises."""
    import lv_xattn_b200 as lvx
    from lv_xattn_b200 import hf_patch, ring
    for mode in ("lv_xattn", "ring", "ring_self"):
        assert callable(hf_patch.patch_cross_attention_forward(mode))
        assert callable(hf_patch.patch_self_attention_forward(mode))
    assert lvx.create_attention_class("ring") is ring.RingAttnFunc
    with pytest.raises(NotImplementedError):
        hf_patch.patch_cross_attention_forward("ulysses")
    with pytest.raises(NotImplementedError):
        lvx.create_attention_class("ulysses")
