"""The real step loop + P2P layer on gloo CPU ranks (world sizes 1-4, odd sizes included), with the kernels
replaced by the tests-only torch stub. Checks slab layout, slot parity, result ownership and the schedule
against the full-tensor oracle, sharded as reference test.py:164-178."""
import math
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCALE = 1.0 / math.sqrt(128.0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    import _stub_ops
    import lv_xattn_b200.attn as attn
    from lv_xattn_b200 import async_communication as ac
    from oracle import attention_oracle as orc
    attn.ops = _stub_ops
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ac.initialize_distributed()
    try:
        B, Hq, Hkv, Sq, Skv, dtype, kv_valid, kw = case
        kw = dict(kw)
        q, k, v, do = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 11, dtype)
        full_bias = None
        if kw.pop("bias", False):
            # the reference's protocol: a KV-side argument stays with the shard, a Q-side argument travels with the
            # query block, and bias_func builds the step's [B, 1, Sq_l, Skv_l] tile from both (test.py:273-286)
            gb = torch.Generator().manual_seed(99)
            key_term = torch.randn(Skv, generator=gb)
            key_term[1::7] = float("-inf")                      # a mask expressed through the bias
            qry_term = torch.randn(Sq, generator=gb)
            full_bias = (qry_term[:, None] + key_term[None, :])[None, None].expand(B, 1, Sq, Skv)
            n, m = Sq // world, Skv // world
            kv_side = [key_term[rank * m:(rank + 1) * m].clone()]
            q_side = [qry_term[rank * n:(rank + 1) * n].clone()]
            if kw.get("baseline") == "ring":                    # there the travelling arguments belong to the K/V shard
                kw.update(bias_func=lambda qa, ka: (qa[:, None] + ka[None, :])[None, None].expand(B, 1, -1, -1),
                          local_bias_args=q_side, remote_bias_args=kv_side)
            else:
                kw.update(bias_func=lambda ka, qa: (qa[:, None] + ka[None, :])[None, None].expand(B, 1, -1, -1),
                          local_bias_args=kv_side, remote_bias_args=q_side)
        o_ref, lse_ref, dq_ref, dk_ref, dv_ref = orc.attention_fwd_bwd(q, k, v, do, SCALE, kv_valid, bias=full_bias)
        ql, dol = orc.shard(q, rank, world), orc.shard(do, rank, world)
        kl, vl = orc.shard(k, rank, world), orc.shard(v, rank, world)
        mod = attn
        if kw.pop("baseline", None) == "ring":      # the K/V-rotating baseline on the same (stubbed) kernels
            from lv_xattn_b200 import ring
            ring.ops = _stub_ops
            mod = ring
        for rep in range(2):   # twice: pooled slabs are reused
            _, _, _, o, L = mod._attn_forward(ql, kl, vl, False, SCALE, None, kv_valid_len=kv_valid, **kw)
            dq, dk, dv = mod._attn_backward(dol, ql, kl, vl, o, L, False, SCALE, None, "flash",
                                            kv_valid_len=kv_valid, **kw)
        tol = 1e-4 if dtype == torch.float32 else 3e-2
        Sl = Sq // world
        lse_l = orc.shard(lse_ref.unsqueeze(-1), rank, world).squeeze(-1)
        L3 = L.view(B, Hq, Sl)
        fin = torch.isfinite(lse_l)
        errs = {
            "o": (o.float() - orc.shard(o_ref, rank, world)).abs().max().item(),
            "lse": (L3[fin] - lse_l[fin]).abs().max().item() if fin.any() else 0.0,
            "dq": (dq.float() - orc.shard(dq_ref, rank, world)).abs().max().item(),
            "dk": (dk.float() - orc.shard(dk_ref, rank, world)).abs().max().item(),
            "dv": (dv.float() - orc.shard(dv_ref, rank, world)).abs().max().item(),
        }
        assert torch.equal(torch.isfinite(L3), fin)
        assert o.dtype == dtype and dq.dtype == dtype and dk.dtype == dtype and dk.shape == kl.shape
        assert L.shape == (B * Hq, Sl) and L.dtype == torch.float32
        bad = {n: e for n, e in errs.items() if not e <= tol}
        ret[rank] = ("ok", errs) if not bad else ("bad", errs)
    except Exception as e:  # surfaced to the parent
        import traceback
        ret[rank] = ("exc", traceback.format_exc())
    finally:
        dist.destroy_process_group()


def _run(world, case):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    for r in range(world):
        assert r in ret, f"rank {r} returned nothing"
        assert ret[r][0] == "ok", f"rank {r}: {ret[r]}"


@pytest.mark.parametrize("schedule", ["gather", "ring"])
@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_step_loop_fp32(world, schedule):
    if world == 1 and schedule == "ring":
        pytest.skip("one rank has no schedule")
    _run(world, (1, 4, 2, 24 * world, 64 * world, torch.float32, None, {"schedule": schedule}))


def test_step_loop_bf16_gqa_key_padding():
    # per-sample valid lengths: one sample ends inside rank 1's shard, one has nothing beyond rank 0
    _run(4, (2, 4, 1, 32, 256, torch.bfloat16, [200, 40], {}))
    _run(4, (2, 4, 1, 32, 256, torch.bfloat16, [200, 40], {"schedule": "ring"}))


@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_ring_baseline_fp32(world):
    """lv_xattn_b200.ring (K/V rotate, dK/dV accumulators travel) against the full-tensor oracle."""
    _run(world, (1, 4, 2, 24 * world, 64 * world, torch.float32, None, {"baseline": "ring"}))


def test_ring_baseline_bf16_gqa_key_padding():
    _run(4, (2, 4, 1, 32, 256, torch.bfloat16, [200, 40], {"baseline": "ring"}))
    _run(2, (1, 2, 2, 32, 128, torch.float32, None, {"baseline": "ring", "no_overlap": True}))


@pytest.mark.parametrize("world", [1, 2, 3])
def test_bias_func_protocol(world):
    """bias_func / local_bias_args / remote_bias_args as in the reference (lv_xattn/attn.py:386-389): the remote
    arguments travel with the query block, the bias tile of every step is built from both, -inf entries mask."""
    _run(world, (1, 4, 2, 16 * world, 48 * world, torch.float32, None, {"bias": True}))


def test_bias_func_protocol_ring_baseline():
    _run(2, (1, 2, 2, 32, 96, torch.float32, None, {"bias": True, "baseline": "ring"}))


def test_step_loop_no_overlap():
    _run(2, (1, 2, 2, 32, 128, torch.float32, None, {"no_overlap": True, "schedule": "ring"}))


def _hf_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    import copy
    import _stub_ops
    import lv_xattn_b200.attn as attn
    from lv_xattn_b200 import async_communication as ac, hf_patch
    from transformers.models.mllama import modeling_mllama as mllama
    attn.ops = _stub_ops
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ac.initialize_distributed()
    try:
        cfg = mllama.MllamaTextConfig(hidden_size=256, num_attention_heads=2, num_key_value_heads=1,
                                      num_hidden_layers=2, intermediate_size=512, vocab_size=64)
        cfg._attn_implementation = "eager"
        torch.manual_seed(0)
        cross = mllama.MllamaTextCrossAttention(cfg, layer_idx=0)
        selfa = mllama.MllamaTextSelfAttention(cfg, layer_idx=1)
        rope = mllama.MllamaRotaryEmbedding(cfg)
        S, Skv = 16 * world, 48 * world
        x = torch.randn(1, S, 256)
        states = torch.randn(1, Skv, 256)
        g = torch.randn(1, S, 256)
        pos = torch.arange(S)[None]
        cos, sin = rope(x, pos)
        causal = torch.full((S, S), float("-inf")).triu(1)[None, None]
        xr = x.clone().requires_grad_(True)
        ref_c, _ = cross(xr, cross_attention_states=states)
        ref_s, _ = selfa(xr, attention_mask=causal, position_embeddings=(cos, sin))
        (ref_c + ref_s).backward(g)
        n, m = S // world, Skv // world
        sl = slice(rank * n, (rank + 1) * n)
        pc, ps = copy.deepcopy(cross), copy.deepcopy(selfa)
        for p_ in list(pc.parameters()) + list(ps.parameters()):
            p_.grad = None
        pc.forward = hf_patch.patch_cross_attention_forward("lv_xattn").__get__(pc)
        ps.forward = hf_patch.patch_self_attention_forward("lv_xattn").__get__(ps)
        xl = x[:, sl].clone().requires_grad_(True)
        hf_patch.set_global_cross_attention_states(states[:, rank * m:(rank + 1) * m].contiguous())
        out_c, _ = pc(xl)
        out_s, _ = ps(xl, attention_mask=None, position_embeddings=(cos[:, sl], sin[:, sl]))
        (out_c + out_s).backward(g[:, sl])
        hf_patch.clear_global_cross_attention_states()
        ok = torch.allclose(out_c, ref_c[:, sl], atol=5e-5, rtol=1e-3) and torch.allclose(out_s, ref_s[:, sl], atol=5e-5, rtol=1e-3)
        ok = ok and torch.allclose(xl.grad, xr.grad[:, sl], atol=1e-4, rtol=1e-3)
        # weight gradients are partial sums per rank: reduce and compare with the unsharded ones
        for (name, p_), (_, pr) in zip(list(pc.named_parameters()) + list(ps.named_parameters()),
                                       list(cross.named_parameters()) + list(selfa.named_parameters())):
            gsum = p_.grad.clone()
            dist.all_reduce(gsum)
            if not torch.allclose(gsum, pr.grad, atol=2e-4, rtol=1e-3):
                ok = False
                ret[rank] = ("bad", name, (gsum - pr.grad).abs().max().item())
        if ok:
            ret[rank] = ("ok",)
        elif rank not in ret:
            ret[rank] = ("bad", "outputs")
    except Exception:
        import traceback
        ret[rank] = ("exc", traceback.format_exc())
    finally:
        dist.destroy_process_group()


def test_hf_hooks_sharded_over_two_ranks():
    pytest.importorskip("transformers.models.mllama.modeling_mllama")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_hf_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        assert ret.get(r, ("missing",))[0] == "ok", f"rank {r}: {ret.get(r)}"


def _late_worker(rank, world, port, ret):
    """Rank 1 shows up three seconds late; rank 0's wait is limited to one second."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    import time
    import _stub_ops
    import lv_xattn_b200.attn as attn
    from lv_xattn_b200 import async_communication as ac
    from oracle import attention_oracle as orc
    attn.ops = _stub_ops
    ac.P2P_TIMEOUT_S = 1.0
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ac.initialize_distributed()
    q, k, v, _ = orc.make_inputs(1, 2, 2, 16 * world, 32 * world, 128, 5, torch.float32)
    ql, kl, vl = (orc.shard(t, rank, world) for t in (q, k, v))
    try:
        if rank == 1:
            time.sleep(3.0)                       # a stalled rank: host-side fault injection only
        t0 = time.perf_counter()
        attn._attn_forward(ql, kl, vl, False, SCALE, None, schedule="ring")
        ret[rank] = ("returned", time.perf_counter() - t0)
    except ac.P2PTimeoutError as e:
        ret[rank] = ("timeout", time.perf_counter() - t0, str(e))
    except Exception as e:  # the late rank may find its peer gone; any error is acceptable for it
        ret[rank] = ("error", type(e).__name__)
    os._exit(0)           # the process group may be wedged by the abandoned transfer: do not try to tear it down


def test_stalled_peer_raises_p2p_timeout():
    """A peer that does not deliver within LVX_P2P_TIMEOUT_S surfaces as P2PTimeoutError on the waiting rank,
    instead of blocking for ever as the reference's wait_async_handles does (async_communication.py:301-305)."""
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_late_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p_ in procs:
        p_.start()
    for p_ in procs:
        p_.join(60)
    for p_ in procs:
        if p_.is_alive():
            p_.kill()
            p_.join()
    assert ret.get(0, ("missing",))[0] == "timeout", dict(ret)
    assert 0.9 <= ret[0][1] <= 2.9, ret[0]          # gave up after about one second, well before rank 1 arrived
    assert "P2P wait exceeded" in ret[0][2]
