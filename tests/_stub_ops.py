"""Tests-only stand-in for lv_xattn_b200.ops so that the step loop, the slab layout and the P2P schedule can run
on gloo CPU ranks. It restates each kernel call with plain torch; it is never importable from the package."""
import torch

from oracle import attention_oracle as orc


class _Part:
    def __init__(self, o, lse, dtype):
        self.o, self.lse, self.dtype = o, lse, dtype


def fwd_partials(q, k, v, sm_scale, kv_valid_len=None, bias=None):
    kvl = None if kv_valid_len is None else [int(x) for x in kv_valid_len]
    if bias is not None:
        o, lse = orc.attention_fwd(q, k, v, sm_scale, kvl, bias=bias)
        return _Part(o, lse.reshape(-1, q.shape[2]), q.dtype)
    if q.dim() == 5:      # [n, B, Hq, Sq, D]: every block against the same K/V
        outs = [orc.attention_fwd(qb, k, v, sm_scale, kvl) for qb in q]
        o = torch.stack([a for a, _ in outs])
        lse = torch.stack([b.reshape(-1, q.shape[-2]) for _, b in outs])
        return _Part(o, lse.reshape(-1, q.shape[-2]), q.dtype)
    o, lse = orc.attention_fwd(q, k, v, sm_scale, kvl)
    return _Part(o, lse.reshape(-1, q.shape[2]), q.dtype)


def fwd_combine(part, o_in, lse_in, o_out, lse_out, final):
    o, lse = part.o, part.lse
    if o_in is not None:
        assert o.dim() == 4
        B, H, S, D = o.shape
        o, lse = orc.merge_partials(o_in, lse_in.view(B, H, S), o, lse.view(B, H, S))
        lse = lse.reshape(-1, S)
    assert o_out.dtype == (part.dtype if final else torch.float32)
    o_out.copy_(o.reshape(o_out.shape))
    lse_out.copy_(lse.reshape(lse_out.shape))


def bwd_prep(o, do):
    S = o.shape[-2]
    return (o.float() * do.float()).sum(-1).reshape(-1, S)


def bwd_block(q, do, lse, delta, k, v, sm_scale, dq_acc, dk_acc, dv_acc, accumulate_dkdv, kv_valid_len=None, bias=None):
    if q.dim() == 5:      # n query blocks, one K/V pass: dK/dV sum over the blocks
        n = q.shape[0]
        rows = lse.numel() // n
        dk32, dv32 = torch.zeros(k.shape), torch.zeros(v.shape)
        for i in range(n):
            bwd_block(q[i], do[i], lse.reshape(n, -1)[i].reshape(-1, q.shape[-2]),
                      delta.reshape(n, -1)[i].reshape(-1, q.shape[-2]), k, v, sm_scale, dq_acc[i], dk32, dv32,
                      True, kv_valid_len)
        if accumulate_dkdv is True:
            dk_acc += dk32
            dv_acc += dv32
        else:
            dk_acc.copy_(dk32)
            dv_acc.copy_(dv32)
        return
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf, dof = q.float(), do.float()
    ke, ve = orc.expand_kv(k.float(), Hq), orc.expand_kv(v.float(), Hq)
    s = torch.matmul(qf, ke.transpose(2, 3)) * sm_scale
    if bias is not None:
        s = s + bias.float()
    if kv_valid_len is not None:
        idx = torch.arange(Skv)[None, None, None, :]
        s = s.masked_fill(idx >= kv_valid_len.view(B, 1, 1, 1).long(), float("-inf"))
    l3 = lse.view(B, Hq, Sq, 1)
    p = torch.where(torch.isinf(l3), torch.zeros_like(s), torch.exp(s - torch.where(torch.isinf(l3), torch.zeros_like(l3), l3)))
    dv = torch.matmul(p.transpose(2, 3), dof)
    dp = torch.matmul(dof, ve.transpose(2, 3))
    ds = p * (dp - delta.view(B, Hq, Sq, 1)) * sm_scale
    dq_acc += torch.matmul(ds, ke)
    dk = torch.matmul(ds.transpose(2, 3), qf)
    dk = dk.view(B, Hkv, g, Skv, D).sum(2)
    dv = dv.view(B, Hkv, g, Skv, D).sum(2)
    if accumulate_dkdv is True:
        dk_acc += dk
        dv_acc += dv
    else:
        dk_acc.copy_(dk)
        dv_acc.copy_(dv)


def add_cast(a, b, out_dtype, out=None):
    r = a if b is None else a + b
    if out is None:
        return r.to(out_dtype)
    out.copy_(r.view(out.shape))
    return out


def fwd_merge_parts(o_parts, lse_parts, out_dtype, o_out=None, lse_out=None):
    n, B, H, S, D = o_parts.shape
    o, lse = o_parts[0], lse_parts[0].view(B, H, S)
    for i in range(1, n):
        o, lse = orc.merge_partials(o, lse, o_parts[i], lse_parts[i].view(B, H, S))
    o, lse = o.to(out_dtype), lse.reshape(B * H, S)
    if o_out is not None:
        o_out.copy_(o)
        lse_out.copy_(lse)
        return o_out, lse_out
    return o, lse


def sum_cast(parts, out_dtype, out=None):
    r = parts.sum(0).to(out_dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


def release_workspaces():
    pass
