"""lvx_kv_project (K/V projection GEMM with the per-head RMSNorm of K fused into its epilogue) and lvx_knorm_bwd
through the C ABI wrappers, against nn.Linear + MllamaTextRMSNorm math in fp32 (reference test_llama3.py:394-419).
Relative Frobenius error of bf16 results against fp32: <= 6e-3 (two roundings: operands are exact, the result is
rounded once; measured ~2e-3)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_project(states, wk, wv, nw, eps, H):
    """fp32: view/transpose as the reference, norm over the head dimension."""
    B, S, hid = states.shape
    x = states.float()
    kpre = (x @ wk.float().t()).view(B, S, H, 128).transpose(1, 2)
    v = (x @ wv.float().t()).view(B, S, H, 128).transpose(1, 2)
    rstd = torch.rsqrt(kpre.pow(2).mean(-1) + eps)
    k = kpre * rstd[..., None] * nw.float()
    return k, v, rstd


def rel(a, b):
    return ((a.float() - b).norm() / b.norm()).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [
    (1, 256, 64, 2),          # one tile, one k-step
    (2, 300, 512, 2),         # rows that cross the batch boundary inside a tile, ragged last tile
    (1, 1601, 4096, 8),       # one image tile of the Llama-3.2-Vision shape: all 8 N tiles, 64 k-steps
    (1, 8192, 1024, 4),       # more tiles than SMs: the persistent loop and the accumulator hand-over
])
def test_kv_project_forward(cuda_device, shape, dtype):
    from lv_xattn_b200 import ops, _lib
    B, S, hid, H = shape
    g = torch.Generator(device=cuda_device).manual_seed(5)
    states = torch.empty(B, S, hid, device=cuda_device).normal_(0, 1, generator=g).to(dtype)
    wk = torch.empty(H * 128, hid, device=cuda_device).normal_(0, 0.02, generator=g).to(dtype)
    wv = torch.empty(H * 128, hid, device=cuda_device).normal_(0, 0.02, generator=g).to(dtype)
    nw = (1 + 0.1 * torch.empty(128, device=cuda_device).normal_(0, 1, generator=g)).to(dtype)
    k, v, rstd = ops.kv_project(states, wk, wv, nw, 1e-5, H)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    k_ref, v_ref, rstd_ref = ref_project(states, wk, wv, nw, 1e-5, H)
    assert k.shape == (B, H, S, 128) and v.shape == (B, H, S, 128) and rstd.shape == (B, H, S)
    assert rel(k, k_ref) <= 6e-3, rel(k, k_ref)
    assert rel(v, v_ref) <= 6e-3, rel(v, v_ref)
    assert rel(rstd, rstd_ref) <= 1e-4, rel(rstd, rstd_ref)
    # without a norm weight K is the plain projection
    k2, _, r2 = ops.kv_project(states, wk, wv, None, 1e-5, H)
    kpre_ref = (states.float() @ wk.float().t()).view(B, S, H, 128).transpose(1, 2)
    assert rel(k2, kpre_ref) <= 6e-3 and torch.equal(r2, torch.ones_like(r2))


def test_kv_project_autograd_matches_modules(cuda_device):
    """KVProjectFunc forward + backward against the same computation through torch modules in fp32: K, V and the
    gradients of both weights, the norm weight and (when asked for) the states."""
    from lv_xattn_b200.projection import KVProjectFunc
    B, S, hid, H = 2, 700, 512, 4
    g = torch.Generator(device=cuda_device).manual_seed(6)
    mk = lambda *sh, std=1.0: torch.empty(*sh, device=cuda_device).normal_(0, std, generator=g)
    states, wk, wv = mk(B, S, hid), mk(H * 128, hid, std=0.05), mk(H * 128, hid, std=0.05)
    nw = 1 + 0.1 * mk(128)
    dk, dv = mk(B, H, S, 128), mk(B, H, S, 128)
    leaves = [t.clone().requires_grad_(True) for t in (states, wk, wv, nw)]
    k_ref, v_ref, _ = ref_project(*leaves, 1e-5, H)
    torch.autograd.backward((k_ref, v_ref), (dk, dv))
    lb = [t.to(torch.bfloat16).requires_grad_(True) for t in (states, wk, wv, nw)]
    k, v = KVProjectFunc.apply(lb[0], lb[1], lb[2], lb[3], 1e-5, H)
    torch.autograd.backward((k, v), (dk.to(torch.bfloat16), dv.to(torch.bfloat16)))
    assert rel(k, k_ref) <= 6e-3 and rel(v, v_ref) <= 6e-3
    for name, a, b in zip(("states", "wk", "wv", "norm_w"), lb, leaves):
        assert a.grad is not None, name
        assert rel(a.grad, b.grad) <= 2e-2, (name, rel(a.grad, b.grad))
