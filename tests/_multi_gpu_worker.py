"""One NCCL rank of tests/test_gpu_multi.py (launched by torch.distributed.run).
argv[1]: comma-separated schedules to run and compare (default "gather,ring")."""
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import torch  # noqa: E402

import _parity  # noqa: E402

import lv_xattn_b200 as lvx  # noqa: E402
from lv_xattn_b200 import _lib  # noqa: E402
from oracle import attention_oracle as orc  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
lvx.initialize_distributed("nccl")
scale = 1.0 / math.sqrt(128.0)
schedules = (sys.argv[1] if len(sys.argv) > 1 else "gather,ring").split(",")
cases = [
    (1, 8, 2, 128 * world, 1024 * world, torch.bfloat16, None),
    (2, 4, 2, 64 * world, 512 * world, torch.bfloat16, [512 * world, 512 * world * 3 // 4]),
    (1, 8, 2, 64 * world, 512 * world, torch.float32, None),
]
for B, Hq, Hkv, Sq, Skv, dtype, valid in cases:
    q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 31, dtype)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = orc.attention_fwd_bwd(q, k, v, do, scale, valid)
    ql, dol, kl, vl = (orc.shard(t, rank, world).to(dev) for t in (q, do, k, v))
    torch.distributed.barrier()          # the oracle above takes a different time on every rank
    for rep, sched in enumerate(schedules):
        if sched == "kvring":       # the K/V-rotating ring baseline on the same kernels (lv_xattn_b200.ring)
            from lv_xattn_b200 import ring
            _, _, _, o, L = ring._attn_forward(ql, kl, vl, False, scale, None, kv_valid_len=valid)
            dq, dk, dv = ring._attn_backward(dol, ql, kl, vl, o, L, False, scale, None, "flash", kv_valid_len=valid)
        elif sched == "hostio":     # pinned host shards through HostStreamedAttention, three pipelined steps (not first)
            st = lvx.HostStreamedAttention(dev)
            hin = [t.cpu().pin_memory() for t in (ql, kl, vl, dol)]
            hout = [torch.empty_like(hin[0]).pin_memory(), torch.empty_like(hin[0]).pin_memory(),
                    torch.empty_like(hin[1]).pin_memory(), torch.empty_like(hin[1]).pin_memory()]
            st.prefetch(*hin)
            for i in range(3):
                if i < 2:
                    st.prefetch(*hin)
                st.step(*hin, scale, *hout, kv_valid_len=valid, wait=False)
            st.finish()
            o, dq, dk, dv = (t.to(dev) for t in hout)
            L = first[1]
        else:
            _, _, _, o, L = lvx._attn_forward(ql, kl, vl, False, scale, None, kv_valid_len=valid, schedule=sched)
            dq, dk, dv = lvx._attn_backward(dol, ql, kl, vl, o, L, False, scale, None, "flash", kv_valid_len=valid,
                                            schedule=sched)
        if rep == 0:
            first = [t.clone() for t in (o, L, dq, dk, dv)]
        for name, a, b in zip(("o", "lse", "dq", "dk", "dv"), first, (o, L, dq, dk, dv)):   # every schedule computes the same thing
            if name == "lse":
                _parity.assert_lse_close(b.cpu(), a.cpu(), f"{sched}_vs_{schedules[0]}", 1e-4)
            elif dtype == torch.float32:
                _parity.assert_fp32(b.cpu(), a.cpu(), name, f"{sched}_vs_{schedules[0]}")
            else:
                _parity.assert_close(b.float().cpu(), a.float().cpu(), name, f"{sched}_vs_{schedules[0]}", *_parity.BF16[name])
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    Sl = Sq // world
    lse_l = orc.shard(lse_ref.unsqueeze(-1), rank, world).squeeze(-1)
    label = f"w{world}_r{rank}_{dtype}"
    got = {"o": o.float().cpu(), "dq": dq.float().cpu(), "dk": dk.float().cpu(), "dv": dv.float().cpu()}
    ref = {"o": orc.shard(o_ref, rank, world), "dq": orc.shard(dq_ref, rank, world),
           "dk": orc.shard(dk_ref, rank, world), "dv": orc.shard(dv_ref, rank, world)}
    _parity.assert_lse_close(L.cpu().view(B, Hq, Sl), lse_l, label, 1e-4 if dtype == torch.float32 else 1e-3)
    for name in got:
        if dtype == torch.float32:
            _parity.assert_fp32(got[name], ref[name], name, label)
        else:
            _parity.assert_close(got[name], ref[name], name, label, *_parity.BF16[name])

# ---- the two Hugging Face hooks on GPU ranks: sharded text and visual sequences against the unsharded stock modules
try:
    from transformers.models.mllama import modeling_mllama as mllama
except ImportError:
    mllama = None
if mllama is not None and "hf" in sys.argv[2:]:
    import copy
    from lv_xattn_b200 import hf_patch
    cfg = mllama.MllamaTextConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                                  num_hidden_layers=2, intermediate_size=512, vocab_size=64)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)                                      # the same weights and inputs on every rank
    cross = mllama.MllamaTextCrossAttention(cfg, layer_idx=0).to(dev)
    selfa = mllama.MllamaTextSelfAttention(cfg, layer_idx=1).to(dev)
    rope = mllama.MllamaRotaryEmbedding(cfg).to(dev)
    S, Skv = 64 * world, 1601 * world                          # per-rank K/V length not a multiple of 128
    x = torch.randn(1, S, 512, device=dev)
    states = torch.randn(1, Skv, 512, device=dev)
    g = torch.randn(1, S, 512, device=dev)
    cos, sin = rope(x, torch.arange(S, device=dev)[None])
    causal = torch.full((S, S), float("-inf"), device=dev).triu(1)[None, None]
    xr = x.clone().requires_grad_(True)
    ref_c, _ = cross(xr, cross_attention_states=states)
    ref_s, _ = selfa(xr, attention_mask=causal, position_embeddings=(cos, sin))
    (ref_c + ref_s).backward(g)
    n, m = S // world, Skv // world
    sl = slice(rank * n, (rank + 1) * n)
    pc, ps = copy.deepcopy(cross).to(torch.bfloat16), copy.deepcopy(selfa).to(torch.bfloat16)
    for p_ in list(pc.parameters()) + list(ps.parameters()):
        p_.grad = None
    pc.forward = hf_patch.patch_cross_attention_forward("lv_xattn").__get__(pc)
    ps.forward = hf_patch.patch_self_attention_forward("lv_xattn").__get__(ps)
    xl = x[:, sl].to(torch.bfloat16).requires_grad_(True)
    hf_patch.set_global_cross_attention_states(states[:, rank * m:(rank + 1) * m].to(torch.bfloat16).contiguous())
    out_c, _ = pc(xl)
    out_s, _ = ps(xl, attention_mask=None,                      # this rank's slice of the rotary tables
                  position_embeddings=(cos[:, sl].to(torch.bfloat16), sin[:, sl].to(torch.bfloat16)))
    (out_c + out_s).backward(g[:, sl].to(torch.bfloat16))
    hf_patch.clear_global_cross_attention_states()

    def rel(a, b):
        return ((a.float() - b).norm() / b.norm()).item()

    assert rel(out_c, ref_c[:, sl]) <= 2e-2 and rel(out_s, ref_s[:, sl]) <= 2e-2, (rel(out_c, ref_c[:, sl]), rel(out_s, ref_s[:, sl]))
    assert rel(xl.grad, xr.grad[:, sl]) <= 3e-2, rel(xl.grad, xr.grad[:, sl])
    for (name, p_), (_, pr) in zip(list(pc.named_parameters()) + list(ps.named_parameters()),
                                   list(cross.named_parameters()) + list(selfa.named_parameters())):
        gsum = p_.grad.float().clone()                          # weight gradients are partial sums per rank
        torch.distributed.all_reduce(gsum)
        assert rel(gsum, pr.grad) <= 3e-2, (name, rel(gsum, pr.grad))
print(f"RANK_OK {rank}", flush=True)
torch.distributed.destroy_process_group()
