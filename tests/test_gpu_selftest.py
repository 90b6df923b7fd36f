"""Tensor-core building blocks: every operand arrangement the attention kernels use, as one 128 x N x K
product through the C ABI (lvx_selftest_mma), against an fp32 matmul of the same rounded inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu

# mode -> (dtype, K, N, a_layout, b_layout); layouts: "mk"/"km" for A, "nk"/"kn" for B
MODES = {
    0: (torch.bfloat16, 128, 128, "mk", "nk"),
    1: (torch.bfloat16, 128, 128, "mk", "kn"),
    2: (torch.bfloat16, 128, 64, "km", "kn"),
    3: (torch.bfloat16, 128, 64, "mk", "nk"),
    4: (torch.bfloat16, 64, 128, "mk", "kn"),
    5: (torch.float32, 64, 128, "mk", "nk"),
    6: (torch.float32, 32, 128, "mk", "kn"),
    7: (torch.float32, 32, 64, "km", "kn"),
}


def run_mode(mode, device):
    from lv_xattn_b200 import ops
    dtype, K, N, la, lb = MODES[mode]
    g = torch.Generator().manual_seed(100 + mode)
    a = torch.randn(128, K, generator=g).to(dtype)   # logical [M, K]
    b = torch.randn(K, N, generator=g).to(dtype)     # logical [K, N]
    ref = a.float() @ b.float()
    a_dev = (a if la == "mk" else a.t().contiguous()).to(device)
    b_dev = (b if lb == "kn" else b.t().contiguous()).to(device)
    d = ops.selftest_mma(mode, a_dev, b_dev, N)
    torch.cuda.synchronize()
    return d.cpu(), ref


@pytest.mark.parametrize("mode", sorted(MODES))
def test_selftest_mode(mode, cuda_device):
    from lv_xattn_b200 import _lib
    d, ref = run_mode(mode, cuda_device)
    assert _lib.device_status() == 0
    # bf16 operands are exact in the product, so only fp32 accumulation order differs;
    # tf32 drops 13 mantissa bits of each operand: |err| <~ K * 2^-11 * |a||b|
    tol = 1e-3 if MODES[mode][0] == torch.bfloat16 else 0.15
    err = (d - ref).abs().max().item()
    assert err < tol, f"mode {mode}: max |err| {err}"
