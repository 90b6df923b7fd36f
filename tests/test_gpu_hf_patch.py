"""The cross-attention hook with the real kernels on one GPU (bf16), and the self-attention hook on one GPU
(bf16), each against the stock Mllama module in fp32 (reference test_llama3.py:263-468)."""
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


def test_self_attention_hook_bf16(cuda_device):
    """patch_self_attention_forward on a GPU rank (W = 1) in bf16 against the stock MllamaTextSelfAttention in fp32
    with an explicit causal mask: outputs and the gradients of the hidden states and of every weight."""
    from lv_xattn_b200 import hf_patch
    cfg = mllama.MllamaTextConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                                  num_hidden_layers=2, intermediate_size=512, vocab_size=64)
    cfg._attn_implementation = "eager"
    torch.manual_seed(1)
    ref_mod = mllama.MllamaTextSelfAttention(cfg, layer_idx=1).to(cuda_device)
    rope = mllama.MllamaRotaryEmbedding(cfg).to(cuda_device)
    mod = copy.deepcopy(ref_mod).to(torch.bfloat16)
    mod.forward = hf_patch.patch_self_attention_forward("lv_xattn").__get__(mod)
    S = 160
    x = torch.randn(2, S, 512, device=cuda_device)
    pos = torch.arange(S, device=cuda_device)[None].expand(2, -1)
    cos, sin = rope(x, pos)
    causal = torch.full((S, S), float("-inf"), device=cuda_device).triu(1)[None, None].expand(2, 1, -1, -1)
    xr = x.clone().requires_grad_(True)
    ref, _ = ref_mod(xr, attention_mask=causal, position_embeddings=(cos, sin))
    g = torch.randn_like(ref)
    ref.backward(g)
    xb = x.to(torch.bfloat16).requires_grad_(True)
    out, _ = mod(xb, attention_mask=None, position_embeddings=(cos.to(torch.bfloat16), sin.to(torch.bfloat16)))
    out.backward(g.to(torch.bfloat16))

    def rel(a, b):
        return ((a.float() - b).norm() / b.norm()).item()

    assert rel(out, ref) <= 2e-2, rel(out, ref)
    assert rel(xb.grad, xr.grad) <= 3e-2, rel(xb.grad, xr.grad)
    for (n, p), (_, pr) in zip(mod.named_parameters(), ref_mod.named_parameters()):
        assert p.grad is not None, n
        assert rel(p.grad, pr.grad) <= 3e-2, (n, rel(p.grad, pr.grad))
