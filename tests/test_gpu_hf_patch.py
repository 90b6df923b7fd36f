"""The cross-attention hook with the real kernels on one GPU (bf16), against the stock Mllama module in fp32."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu
mllama = pytest.importorskip("transformers.models.mllama.modeling_mllama")


def test_cross_attention_hook_bf16(cuda_device):
    from lv_xattn_b200 import hf_patch
    cfg = mllama.MllamaTextConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                                  num_hidden_layers=2, intermediate_size=512, vocab_size=64)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    ref_mod = mllama.MllamaTextCrossAttention(cfg, layer_idx=0).to(cuda_device)
    mod = copy.deepcopy(ref_mod).to(torch.bfloat16)
    mod.forward = hf_patch.patch_cross_attention_forward("lv_xattn").__get__(mod)
    x = torch.randn(1, 192, 512, device=cuda_device)
    states = torch.randn(1, 1601, 512, device=cuda_device)          # one image tile's tokens: a ragged K/V length
    xr = x.clone().requires_grad_(True)
    ref, _ = ref_mod(xr, cross_attention_states=states)
    g = torch.randn_like(ref)
    ref.backward(g)
    xb = x.to(torch.bfloat16).requires_grad_(True)
    hf_patch.set_global_cross_attention_states(states.to(torch.bfloat16))
    try:
        out, _ = mod(xb)
        out.backward(g.to(torch.bfloat16))
    finally:
        hf_patch.clear_global_cross_attention_states()
    scale = ref.abs().max().item()
    assert (out.float() - ref).abs().max().item() <= 3e-2 * max(1.0, scale)
    gs = xr.grad.abs().max().item()
    assert (xb.grad.float() - xr.grad).abs().max().item() <= 5e-2 * max(1.0, gs)
    for (n, p), (_, pr) in zip(mod.named_parameters(), ref_mod.named_parameters()):
        assert p.grad is not None, n
        tol = 5e-2 * max(1.0, pr.grad.abs().max().item())
        assert (p.grad.float() - pr.grad).abs().max().item() <= tol, n
