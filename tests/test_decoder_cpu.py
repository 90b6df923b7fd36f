"""A whole (tiny) Mllama text decoder -- self-attention layers, gated cross-attention layers, embeddings, head, loss --
with both hooks installed on the Hugging Face classes (as reference test_llama3.py:666-667 does), the text sequence and
the visual states sharded over two gloo ranks, against the same model unsharded with the stock forwards. The kernels
are the tests-only torch stub; what is checked is everything around them: per-rank positions for the rotary tables,
the global causal mask of the self-attention hook, K/V recompute, gradient flow into every parameter."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytest.importorskip("transformers.models.mllama.modeling_mllama")


def build(seed=0):
    from transformers.models.mllama import modeling_mllama as M
    cfg = M.MllamaTextConfig(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, num_hidden_layers=4,
                             intermediate_size=512, vocab_size=96, cross_attention_layers=[1, 3], rms_norm_eps=1e-5,
                             max_position_embeddings=512, pad_token_id=0)
    cfg._attn_implementation = "eager"
    torch.manual_seed(seed)
    model = M.MllamaForCausalLM(cfg)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "gate" in n:
                p.fill_(0.7)                  # the stock init is 0: cross-attention would contribute nothing
    return model


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    import _stub_ops
    import lv_xattn_b200.attn as attn
    from lv_xattn_b200 import async_communication as ac, hf_patch
    attn.ops = _stub_ops
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ac.initialize_distributed()
    try:
        S, Skv = 16 * world, 40 * world
        g = torch.Generator().manual_seed(5)
        ids = torch.randint(1, 96, (1, S), generator=g)
        labels = torch.randint(1, 96, (1, S), generator=g)
        states = torch.randn(1, Skv, 256, generator=g)
        # ---- unsharded, stock forwards
        ref = build()
        h_ref = ref.model(input_ids=ids, cross_attention_states=states, use_cache=False).last_hidden_state
        logits = ref.lm_head(h_ref).float()
        loss_ref = torch.nn.functional.cross_entropy(logits.view(-1, 96), labels.view(-1), reduction="sum")
        loss_ref.backward()
        # ---- sharded, hooks installed
        model = build()
        hf_patch.install_hooks("lv_xattn")
        try:
            n, m = S // world, Skv // world
            sl = slice(rank * n, (rank + 1) * n)
            pos = (torch.arange(n) + rank * n)[None]
            h = model.model(input_ids=ids[:, sl], position_ids=pos, use_cache=False,       # training path: no KV cache
                            cross_attention_states=states[:, rank * m:(rank + 1) * m].contiguous()).last_hidden_state
            lg = model.lm_head(h).float()
            loss = torch.nn.functional.cross_entropy(lg.view(-1, 96), labels[:, sl].reshape(-1), reduction="sum")
            loss.backward()
        finally:
            hf_patch.uninstall_hooks()
            hf_patch.clear_global_cross_attention_states()
        ok = torch.allclose(h, h_ref[:, sl], atol=2e-4, rtol=1e-3)
        tot = loss.detach().clone()
        dist.all_reduce(tot)
        ok = ok and abs(tot.item() - loss_ref.item()) <= 1e-3 * abs(loss_ref.item())
        bad = None
        for (name, p), (_, pr) in zip(model.named_parameters(), ref.named_parameters()):
            gsum = (p.grad if p.grad is not None else torch.zeros_like(p)).clone()
            dist.all_reduce(gsum)                       # replicated weights: the ranks' gradients add up
            err = (gsum - pr.grad).norm().item()
            if err > 1e-3 * pr.grad.norm().item() + 1e-6:       # fp32 summation order only
                bad = (name, err, pr.grad.norm().item())
                break
        ret[rank] = ("ok",) if ok and bad is None else ("bad", ok, bad)
    except Exception:
        import traceback
        ret[rank] = ("exc", traceback.format_exc())
    finally:
        dist.destroy_process_group()


def test_sharded_decoder_matches_unsharded():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        assert ret.get(r, ("missing",))[0] == "ok", f"rank {r}: {ret.get(r)}"
