"""Ring attention (the K/V-rotating baseline) on the same kernels as the LV-XAttn path.

The reference ships this scheme as its comparison baseline (`ring/attn.py`: `_attn_forward` :190-283,
`_attn_backward` :285-388) and as `attention_mode="ring"` of its drivers (test.py:255, test_llama3.py:107). Here it is
the same schedule on this library's block kernels, so that the two schemes can be timed against each other on equal
kernels:

  forward   Q, O and the softmax statistics stay at home; the K/V shards travel rank -> rank+1 (W-1 hops). Each step
            runs the forward block against the visiting shard and merges into the local (O, lse) accumulator.
  backward  K/V travel again, each shard together with its fp32 dK/dV accumulator, which every rank adds to and which
            returns home with the W-th hop; dQ accumulates locally in fp32.

Per GPU and direction the ring moves (W-1) K/V shards forward and (W-1) K/V shards plus W fp32 dK/dV shards backward --
bytes that grow with the visual sequence, where LV-XAttn moves the (short) query side only. Same signatures, key-padding
argument and return conventions as `lv_xattn_b200.attn`.
"""
from __future__ import annotations

import torch

from . import ops
from .async_communication import (
    _exchange,
    get_sequence_parallel_rank,
    get_sequence_parallel_size,
    get_slabs,
    wait_async_handles,
)
from .attn import _build_bias, _carve, _check_common


def _visiting_valid(kv_valid_len, home: int, skv_local: int, device):
    """Key-padding clamp of the shard whose home is rank `home` (see attn._local_valid)."""
    if kv_valid_len is None:
        return None
    t = torch.as_tensor(kv_valid_len, device=device).to(torch.int64)
    return (t - home * skv_local).clamp_(0, skv_local).to(torch.int32).contiguous()


def _attn_forward(q, k, v, causal, sm_scale, comm_mode, bias_func=None, local_bias_args=[], remote_bias_args=[],
                  no_overlap=False, kv_valid_len=None):
    """Returns (q, k, v, o, L) like lv_xattn_b200.attn._attn_forward (reference ring/attn.py:190-283)."""
    _check_common(q, k, v, causal, bias_func, local_bias_args, remote_bias_args)
    W, rank = get_sequence_parallel_size(), get_sequence_parallel_rank()
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dev, dt = q.device, q.dtype
    es = q.element_size()
    qc = q.contiguous()
    n_kv = B * Hkv * Skv * D
    o = torch.empty(B, Hq, Sq, D, dtype=dt, device=dev)
    L = torch.empty(B * Hq, Sq, dtype=torch.float32, device=dev)
    steps = 1 if (W == 1 or comm_mode == "nocomm") else W
    # visiting shard: [K | V] in one slab, two slabs alternate
    bufs = get_slabs("ring_kv", 2 * n_kv * es, dev, 2)
    acc = get_slabs("ring_fwd_acc", (B * Hq * Sq * D + B * Hq * Sq) * 4, dev, 2)

    def kv_views(buf):
        return _carve(buf, 0, (B, Hkv, Skv, D), dt), _carve(buf, n_kv * es, (B, Hkv, Skv, D), dt)

    def acc_views(buf):
        return (_carve(buf, 0, (B, Hq, Sq, D), torch.float32),
                _carve(buf, B * Hq * Sq * D * 4, (B * Hq, Sq), torch.float32))

    cur = bufs[0]
    ck, cv = kv_views(cur)
    ck.copy_(k)
    cv.copy_(v)
    # with a bias_func the "remote" arguments belong to the K/V shard and travel with it (reference
    # ring/attn.py:246-258); the local ones belong to the queries
    args_cur = [a.contiguous() for a in remote_bias_args] if bias_func is not None else []
    args_bufs = [[torch.empty_like(a) for a in args_cur] for _ in range(2)]
    reqs = []
    o_in = l_in = None
    for t in range(steps):
        last = t == steps - 1
        wait_async_handles(reqs)                     # the shard this step works on has arrived
        reqs = []
        ck, cv = kv_views(cur)
        if not last:
            nxt = bufs[(t + 1) % 2]
            args_next = args_bufs[t % 2]
            reqs = _exchange([cur[:2 * n_kv * es], *args_cur], [nxt[:2 * n_kv * es], *args_next], comm_mode)
            if no_overlap:
                wait_async_handles(reqs)
                reqs = []
        kvl = _visiting_valid(kv_valid_len, (rank - t) % W, Skv, dev)
        bias = _build_bias(bias_func, local_bias_args, args_cur, qc, ck)
        part = ops.fwd_partials(qc, ck, cv, sm_scale, kvl, bias=bias)
        o_out, l_out = (o, L) if last else acc_views(acc[t % 2])
        ops.fwd_combine(part, o_in, l_in, o_out, l_out, last)
        o_in, l_in = o_out, l_out
        if not last:
            cur, args_cur = nxt, args_next
    wait_async_handles(reqs)
    return q, k, v, o, L


def _attn_backward(do, q, k, v, o, L, causal, sm_scale, comm_mode, backward_engine, bias_func=None,
                   local_bias_args=[], remote_bias_args=[], no_overlap=False, kv_valid_len=None):
    """Returns (dq, dk, dv) like lv_xattn_b200.attn._attn_backward (reference ring/attn.py:285-388)."""
    _check_common(q, k, v, causal, bias_func, local_bias_args, remote_bias_args)
    W, rank = get_sequence_parallel_size(), get_sequence_parallel_rank()
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dev, dt = q.device, q.dtype
    es = q.element_size()
    qc, oc, doc = q.contiguous(), o.contiguous(), do.contiguous()
    if L.dtype != torch.float32 or L.numel() != B * Hq * Sq:
        raise ValueError("L must be the fp32 [B*Hq, Sq] log-sum-exp returned by _attn_forward")
    Lc = L.contiguous().view(B * Hq, Sq)
    n_q, n_kv = B * Hq * Sq * D, B * Hkv * Skv * D
    delta = ops.bwd_prep(oc, doc)
    dq_acc = _carve(get_slabs("ring_dq", n_q * 4, dev, 1)[0], 0, (B, Hq, Sq, D), torch.float32)
    dq_acc.zero_()
    dq = torch.empty(B, Hq, Sq, D, dtype=dt, device=dev)
    if W == 1 or comm_mode == "nocomm":
        dk = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        dv = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        kvl = _visiting_valid(kv_valid_len, rank, Skv, dev)
        bias = _build_bias(bias_func, local_bias_args, remote_bias_args, qc, k)
        ops.bwd_block(qc, doc, Lc, delta, k.contiguous(), v.contiguous(), sm_scale, dq_acc, dk, dv, "final", kvl,
                      bias=bias)
        ops.add_cast(dq_acc, None, dt, out=dq)
        return dq, dk, dv

    kv_bufs = get_slabs("ring_kv", 2 * n_kv * es, dev, 2)
    g_bufs = get_slabs("ring_dkdv", 2 * n_kv * 4, dev, 2)     # travelling fp32 [dK | dV] of the visiting shard

    def kv_views(buf):
        return _carve(buf, 0, (B, Hkv, Skv, D), dt), _carve(buf, n_kv * es, (B, Hkv, Skv, D), dt)

    def g_views(buf):
        return (_carve(buf, 0, (B, Hkv, Skv, D), torch.float32),
                _carve(buf, n_kv * 4, (B, Hkv, Skv, D), torch.float32))

    cur = kv_bufs[0]
    ck, cv = kv_views(cur)
    ck.copy_(k)
    cv.copy_(v)
    kv_reqs, g_reqs = [], []
    args_cur = [a.contiguous() for a in remote_bias_args] if bias_func is not None else []
    args_bufs = [[torch.empty_like(a) for a in args_cur] for _ in range(2)]
    for t in range(W):
        last = t == W - 1
        wait_async_handles(kv_reqs)
        kv_reqs = []
        ck, cv = kv_views(cur)
        if not last:
            nxt = kv_bufs[(t + 1) % 2]
            args_next = args_bufs[t % 2]
            kv_reqs = _exchange([cur[:2 * n_kv * es], *args_cur], [nxt[:2 * n_kv * es], *args_next], comm_mode)
            if no_overlap:
                wait_async_handles(kv_reqs)
                kv_reqs = []
        # The accumulator of the visiting shard: fresh at step 0 (it is this rank's own shard), otherwise what
        # rank-1 sent after its previous step, which lands in g_bufs[t % 2].
        wait_async_handles(g_reqs)
        g_reqs = []
        gk, gv = g_views(g_bufs[t % 2])
        kvl = _visiting_valid(kv_valid_len, (rank - t) % W, Skv, dev)
        bias = _build_bias(bias_func, local_bias_args, args_cur, qc, ck)
        ops.bwd_block(qc, doc, Lc, delta, ck, cv, sm_scale, dq_acc, gk, gv, t > 0, kvl, bias=bias)
        # on to rank+1 (after the last step this is the hop that brings every finished accumulator home)
        g_reqs = _exchange([g_bufs[t % 2][:2 * n_kv * 4]], [g_bufs[(t + 1) % 2][:2 * n_kv * 4]], comm_mode)
        if no_overlap:
            wait_async_handles(g_reqs)
            g_reqs = []
        if not last:
            cur, args_cur = nxt, args_next
    wait_async_handles(g_reqs)
    gk, gv = g_views(g_bufs[W % 2])
    dk = ops.add_cast(gk, None, dt)
    dv = ops.add_cast(gv, None, dt)
    ops.add_cast(dq_acc, None, dt, out=dq)
    return dq, dk, dv


class RingAttnFunc(torch.autograd.Function):
    """attention(q, k, v, causal, sm_scale, ...) -> o with the ring schedule; same call shape as attn.LVXAttnFunc
    (the class reference test.py:38-77 builds for attention_mode="ring")."""

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, bias_func=None, local_bias_args=[], remote_bias_args=[],
                kv_valid_len=None):
        q, k, v, o, L = _attn_forward(q, k, v, causal, sm_scale, None, bias_func=bias_func,
                                      local_bias_args=local_bias_args, remote_bias_args=remote_bias_args,
                                      kv_valid_len=kv_valid_len)
        ctx.save_for_backward(q, k, v, o, L)
        ctx.sm_scale, ctx.causal, ctx.kv_valid_len = sm_scale, causal, kv_valid_len
        ctx.bias = (bias_func, local_bias_args, remote_bias_args)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, L = ctx.saved_tensors
        bias_func, local_bias_args, remote_bias_args = ctx.bias
        dq, dk, dv = _attn_backward(do, q, k, v, o, L, ctx.causal, ctx.sm_scale, None, "flash", bias_func=bias_func,
                                    local_bias_args=local_bias_args, remote_bias_args=remote_bias_args,
                                    kv_valid_len=ctx.kv_valid_len)
        return dq, dk, dv, None, None, None, None, None, None
