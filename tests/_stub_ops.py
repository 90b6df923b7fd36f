"""Tests-only stand-in for lv_xattn_b200.ops so that the step loop, the slab layout and the P2P schedule can run
on gloo CPU ranks. It restates each kernel call with plain torch; it is never importable from the package."""
import torch

from oracle import attention_oracle as orc


class _Part:
    def __init__(self, o, lse, dtype):
        self.o, self.lse, self.dtype = o, lse, dtype


def fwd_partials(q, k, v, sm_scale, kv_valid_len=None):
    kvl = None if kv_valid_len is None else [int(x) for x in kv_valid_len]
    o, lse = orc.attention_fwd(q, k, v, sm_scale, kvl)
    return _Part(o, lse.reshape(-1, q.shape[2]), q.dtype)


def fwd_combine(part, o_in, lse_in, o_out, lse_out, final):
    o, lse = part.o, part.lse
    if o_in is not None:
        B, H, S, D = o.shape
        o, lse = orc.merge_partials(o_in, lse_in.view(B, H, S), o, lse.view(B, H, S))
        lse = lse.reshape(-1, S)
    assert o_out.dtype == (part.dtype if final else torch.float32)
    o_out.copy_(o)
    lse_out.copy_(lse)


def bwd_prep(o, do):
    B, H, S, D = o.shape
    return (o.float() * do.float()).sum(-1).reshape(B * H, S)


def bwd_block(q, do, lse, delta, k, v, sm_scale, dq_acc, dk_acc, dv_acc, accumulate_dkdv, kv_valid_len=None):
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf, dof = q.float(), do.float()
    ke, ve = orc.expand_kv(k.float(), Hq), orc.expand_kv(v.float(), Hq)
    s = torch.matmul(qf, ke.transpose(2, 3)) * sm_scale
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
    if accumulate_dkdv:
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


def release_workspaces():
    pass
