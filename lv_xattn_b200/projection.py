"""K/V projection of the visual states for the patched cross-attention layer.

The reference's `project()` closure (test_llama3.py:394-419) runs k_proj and v_proj on the visual states, reshapes
and transposes both to [B, H, S, D], expands them to the query head count and applies k_norm -- as separate torch
modules, in forward and again in the backward recompute. At the Llama-3.2-Vision shapes these GEMMs cost about as much
as the attention itself. `KVProjectFunc` is the same computation as ONE tensor-core GEMM with the per-head RMSNorm
fused into its epilogue and the result written directly in the [B, Hkv, S, 128] layout the attention kernels read
(`lvx_kv_project`). Its backward keeps the weight gradients on library GEMMs (torch.matmul): the norm's backward is
one small kernel of this library (`lvx_knorm_bwd`), then dWk = dKpre^T X and dWv = dV^T X per head, reading dK/dV in
place (no transposed copies). The states get a gradient only if they ask for one.
"""
from __future__ import annotations

import torch

from . import ops


class KVProjectFunc(torch.autograd.Function):
    """(states [B,S,hidden], wk, wv [Hkv*128, hidden], norm_weight [128], eps, n_kv_heads) -> (K, V) [B,Hkv,S,128]."""

    @staticmethod
    def forward(ctx, states, wk, wv, norm_weight, eps, n_kv_heads):
        k, v, rstd = ops.kv_project(states, wk, wv, norm_weight, eps, n_kv_heads)
        ctx.save_for_backward(states, wk, wv, norm_weight, k, rstd)
        ctx.n_kv_heads = n_kv_heads
        return k, v

    @staticmethod
    def backward(ctx, dk, dv):
        states, wk, wv, norm_weight, k, rstd = ctx.saved_tensors
        H = ctx.n_kv_heads
        B, S, hid = states.shape
        dk, dv = dk.contiguous(), dv.contiguous()
        if norm_weight is not None:
            dkpre, dnw = ops.knorm_bwd(k, dk, rstd, norm_weight)
        else:
            dkpre, dnw = dk, None
        g_wk = g_wv = g_states = g_nw = None
        if ctx.needs_input_grad[1]:
            # dWk[h] = sum_b dKpre[b,h]^T X[b]: [128, S] x [S, hidden]; the transposed operand is read in place
            g_wk = sum(torch.matmul(dkpre[b].transpose(-1, -2), states[b]) for b in range(B)).reshape(H * 128, hid)
        if ctx.needs_input_grad[2]:
            g_wv = sum(torch.matmul(dv[b].transpose(-1, -2), states[b]) for b in range(B)).reshape(H * 128, hid)
        if ctx.needs_input_grad[0]:
            wk3, wv3 = wk.view(H, 128, hid), wv.view(H, 128, hid)
            g_states = (torch.matmul(dkpre, wk3).sum(1) + torch.matmul(dv, wv3).sum(1))
        if norm_weight is not None and ctx.needs_input_grad[3]:
            g_nw = dnw.to(norm_weight.dtype)
        return g_states, g_wk, g_wv, g_nw, None, None


def kv_project(states, wk, wv, norm_weight, eps, n_kv_heads):
    """The fused projection when the tensors qualify (CUDA, bf16/fp16, hidden a multiple of 64, an even number of KV
    heads); None otherwise, and the caller keeps its own modules."""
    if not ops.kv_project_supported(states, wk, wv, n_kv_heads):
        return None
    return KVProjectFunc.apply(states, wk, wv, norm_weight, float(eps), n_kv_heads)
