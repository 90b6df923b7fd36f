"""Hugging Face Mllama hooks: replacements for the `forward` of the text cross-attention and self-attention
modules that run sequence-parallel, as the reference's drivers install them
(test_llama3.py:263-468, assigned onto the HF classes at :666-667).

    from transformers.models.mllama import modeling_mllama as M
    from lv_xattn_b200.hf_patch import patch_cross_attention_forward, patch_self_attention_forward
    M.MllamaTextCrossAttention.forward = patch_cross_attention_forward("lv_xattn")
    M.MllamaTextSelfAttention.forward = patch_self_attention_forward("lv_xattn")

The reference was written against transformers 4.47 (`MllamaText{Cross,Self}SdpaAttention`, 3-tuple returns);
these hooks target the classes of the installed transformers (`MllamaTextCrossAttention` /
`MllamaTextSelfAttention`, 2-tuple returns) and accept both spellings of the cache argument.

Each rank passes its own shard: `hidden_states` holds rows [r*S/W, (r+1)*S/W) of the text sequence and the
cross-attention states rows [r*Skv/W, (r+1)*Skv/W) of the visual sequence. The visual states are taken from a
module global (reference test_llama3.py:69-79) so that autograd holds no reference to them: only
(hidden_states, o, lse) are kept per layer and K/V are re-projected in backward.
Differences from the reference: K/V stay at `num_key_value_heads` (no `repeat_kv`, :416-417); gradients flow into
the hidden states and the projection weights (the reference's wrapper returns None for all of them, :243);
key padding of the visual sequence can be given as `set_global_cross_attention_states(states, kv_valid_len)`.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .async_communication import get_sequence_parallel_group, get_sequence_parallel_rank, get_sequence_parallel_size
from .attn import LVXAttnRecomputeFunc, RingAttnRecomputeFunc
from .projection import kv_project

ATTENTION_MODES = ("lv_xattn", "ring", "ring_self")      # the reference's modes (test_llama3.py:107)

_GLOBAL_CROSS_ATTENTION_STATES = None
_GLOBAL_KV_VALID_LEN = None


def set_global_cross_attention_states(cross_attention_states, kv_valid_len=None):
    """Registers this rank's shard of the visual features [B, Skv_local, hidden] for the cross-attention
    layers of the next forward/backward, with optional GLOBAL valid lengths per batch entry."""
    global _GLOBAL_CROSS_ATTENTION_STATES, _GLOBAL_KV_VALID_LEN
    _GLOBAL_CROSS_ATTENTION_STATES = cross_attention_states
    _GLOBAL_KV_VALID_LEN = kv_valid_len


def get_global_cross_attention_states():
    return _GLOBAL_CROSS_ATTENTION_STATES


def clear_global_cross_attention_states():
    set_global_cross_attention_states(None, None)


def _check_mode(attention_mode):
    if attention_mode not in ATTENTION_MODES:
        raise NotImplementedError(f"attention_mode {attention_mode!r}: expected one of {ATTENTION_MODES}")


def patch_cross_attention_forward(attention_mode="lv_xattn"):
    """Returns an unbound `forward` for `MllamaTextCrossAttention` (reference test_llama3.py:356-468).
    attention_mode "lv_xattn" rotates the query side (K/V resident); "ring" / "ring_self" run the K/V-rotating
    baseline (lv_xattn_b200.ring) on the same kernels."""
    _check_mode(attention_mode)
    recompute = LVXAttnRecomputeFunc if attention_mode == "lv_xattn" else RingAttnRecomputeFunc

    def forward(self, hidden_states, cross_attention_states=None, past_key_values=None, attention_mask=None,
                output_attentions=False, use_cache=None, cache_position=None, past_key_value=None, **kwargs):
        if output_attentions:
            raise NotImplementedError("attention weights are never materialised by the flash kernels")
        if past_key_values is not None or past_key_value is not None:
            raise NotImplementedError("KV caching is a decoding feature; this hook is the training path")
        if cross_attention_states is not None and cross_attention_states is not get_global_cross_attention_states():
            # states handed to the call always win (the model passes fresh ones on every forward, reference
            # test_llama3.py:540); valid lengths registered for other states do not carry over
            set_global_cross_attention_states(cross_attention_states, None)
        if get_global_cross_attention_states() is None:
            raise ValueError("no cross-attention states: pass them or call set_global_cross_attention_states")
        bsz, q_len, _ = hidden_states.size()
        nh, nkv, hd = self.num_heads, self.num_key_value_heads, self.head_dim

        def project(x, states):
            q = self.q_proj(x).view(bsz, q_len, nh, hd).transpose(1, 2)
            q = self.q_norm(q)
            # K/V of the visual states: one fused GEMM with the norm in its epilogue, written in the kernels' layout
            # (projection.KVProjectFunc); the module path is kept for tensors it does not take (CPU, fp32, biases)
            fused = None
            if hd == 128 and self.k_proj.bias is None and self.v_proj.bias is None:
                eps = getattr(self.k_norm, "variance_epsilon", getattr(self.k_norm, "eps", 1e-6))
                fused = kv_project(states, self.k_proj.weight, self.v_proj.weight, self.k_norm.weight, eps, nkv)
            if fused is not None:
                k, v = fused
            else:
                k = self.k_proj(states).view(bsz, -1, nkv, hd).transpose(1, 2)
                v = self.v_proj(states).view(bsz, -1, nkv, hd).transpose(1, 2)
                k = self.k_norm(k).contiguous()
                v = v.contiguous()
            return q.contiguous(), k, v

        params = [p for p in (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight, self.q_norm.weight,
                              self.k_norm.weight)]
        # the states of THIS call are bound here: a second forward with other states before this call's backward
        # must not change what the recompute projects
        states_now = get_global_cross_attention_states()
        attn = recompute.apply(hidden_states, project, False, lambda: states_now, _GLOBAL_KV_VALID_LEN, *params)
        attn = attn.transpose(1, 2).reshape(bsz, q_len, nh * hd).contiguous()
        return self.o_proj(attn), None

    return forward


class _AllGatherSeq(torch.autograd.Function):
    """All-gather along the sequence axis (dim 2) over the sequence-parallel group; backward returns the
    local slice of the summed gradient."""

    @staticmethod
    def forward(ctx, x):
        w = get_sequence_parallel_size()
        parts = [torch.empty_like(x) for _ in range(w)]
        dist.all_gather(parts, x.contiguous(), group=get_sequence_parallel_group())
        return torch.cat(parts, dim=2)

    @staticmethod
    def backward(ctx, g):
        w, r = get_sequence_parallel_size(), get_sequence_parallel_rank()
        g = g.contiguous()
        dist.all_reduce(g, group=get_sequence_parallel_group())
        n = g.shape[2] // w
        return g[:, :, r * n:(r + 1) * n].contiguous()


def patch_self_attention_forward(attention_mode="lv_xattn"):
    """Returns an unbound `forward` for `MllamaTextSelfAttention` (reference test_llama3.py:263-354).

    The text sequence is short next to the visual one (2,048 tokens in the end-to-end configuration), so the
    self-attention layers gather K/V over the sequence-parallel group and apply the causal mask with global
    positions (query row i of rank r sits at position r*S_local + i). `position_embeddings` must already be
    this rank's slice of the rotary tables. The attention itself is torch's scaled_dot_product_attention: the
    self-attention layers are not the path this library accelerates. Every attention_mode gets this
    implementation: the reference's "ring_self" applies its causal mask with rank-local indices at every step
    (ring/attn.py:280), which is not globally correct, so it is not reproduced."""
    _check_mode(attention_mode)

    def forward(self, hidden_states, attention_mask=None, position_embeddings=None, output_attentions=False,
                use_cache=False, past_key_values=None, cache_position=None, past_key_value=None, **kwargs):
        from transformers.models.mllama.modeling_mllama import apply_rotary_pos_emb
        if output_attentions:
            raise NotImplementedError("attention weights are not materialised")
        if past_key_values is not None or past_key_value is not None:
            raise NotImplementedError("KV caching is a decoding feature; this hook is the training path")
        bsz, q_len, _ = hidden_states.size()
        nh, nkv, hd = self.num_heads, self.num_key_value_heads, self.head_dim
        q = self.q_proj(hidden_states).view(bsz, q_len, nh, hd).transpose(1, 2)
        k = self.k_proj(hidden_states).view(bsz, q_len, nkv, hd).transpose(1, 2)
        v = self.v_proj(hidden_states).view(bsz, q_len, nkv, hd).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        w, r = get_sequence_parallel_size(), get_sequence_parallel_rank()
        if w > 1:
            k, v = _AllGatherSeq.apply(k), _AllGatherSeq.apply(v)
        kv_len = k.shape[2]
        qpos = torch.arange(q_len, device=q.device) + r * q_len
        mask = (torch.arange(kv_len, device=q.device)[None, :] <= qpos[:, None])          # [q_len, kv_len]
        out = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask[None, None], scale=self.scaling,
                                                               enable_gqa=nh != nkv)
        out = out.transpose(1, 2).reshape(bsz, q_len, nh * hd).contiguous()
        return self.o_proj(out), None

    return forward


_SAVED_FORWARDS = {}


def install_hooks(attention_mode="lv_xattn"):
    """Assigns the two hooks onto the installed transformers' Mllama text attention classes, as the reference's
    driver does (test_llama3.py:666-667). Every MllamaTextCrossAttention / MllamaTextSelfAttention of every model in
    the process is then sequence-parallel; `uninstall_hooks()` restores the stock forwards."""
    from transformers.models.mllama import modeling_mllama as M
    if not _SAVED_FORWARDS:
        _SAVED_FORWARDS["cross"] = M.MllamaTextCrossAttention.forward
        _SAVED_FORWARDS["self"] = M.MllamaTextSelfAttention.forward
    M.MllamaTextCrossAttention.forward = patch_cross_attention_forward(attention_mode)
    M.MllamaTextSelfAttention.forward = patch_self_attention_forward(attention_mode)


def uninstall_hooks():
    from transformers.models.mllama import modeling_mllama as M
    if _SAVED_FORWARDS:
        M.MllamaTextCrossAttention.forward = _SAVED_FORWARDS.pop("cross")
        M.MllamaTextSelfAttention.forward = _SAVED_FORWARDS.pop("self")
