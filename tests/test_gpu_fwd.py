"""Forward block + combine/merge through the C ABI against the CPU oracle (bf16/fp16 inputs, fp32 oracle on
the same rounded inputs). Tolerances: O max-abs <= 2e-2, lse <= 1e-3 (the stated bf16 bar), plus the relative
criteria of tests/_parity.py (Frobenius <= 1e-2, max error <= 5 % of max|O|) that still bite when |O| << 2e-2."""
import math

import pytest
import torch

import _parity
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128.0)


def run_case(device, B, Hq, Hkv, Sq, Skv, dtype, seed=1, kv_valid=None):
    from lv_xattn_b200 import ops, _lib
    q, k, v, _ = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, seed, dtype)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, SCALE, kv_valid)
    kvl = None if kv_valid is None else torch.tensor(kv_valid, dtype=torch.int32, device=device)
    o, lse = ops.fwd_block(q.to(device), k.to(device), v.to(device), SCALE, kv_valid_len=kvl)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    o, lse = o.float().cpu(), lse.cpu().view(B, Hq, Sq)
    return o, lse, o_ref, lse_ref


def check(o, lse, o_ref, lse_ref, label="fwd"):
    _parity.assert_lse_close(lse, lse_ref, label)
    _parity.assert_close(o, o_ref, "o", label, *_parity.BF16["o"])


@pytest.mark.parametrize("shape", [
    (1, 1, 1, 128, 128),       # one tile
    (1, 2, 1, 128, 256),       # GQA 2 heads -> one 256-row CTA, two K/V tiles
    (1, 4, 1, 64, 1024),       # packed rows cross head boundaries inside a tile
    (2, 8, 2, 192, 2048),      # ragged packed rows (768 = 3 tiles), split-KV
    (1, 32, 8, 512, 8192),     # the reference's correctness shape, 16-bit inputs
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fwd_shapes(cuda_device, shape, dtype):
    B, Hq, Hkv, Sq, Skv = shape
    check(*run_case(cuda_device, B, Hq, Hkv, Sq, Skv, dtype), label=f"fwd{shape}{dtype}")


@pytest.mark.parametrize("skv", [32, 100, 129, 1000, 51232 // 8])
def test_fwd_ragged_kv(cuda_device, skv):
    check(*run_case(cuda_device, 1, 4, 2, 96, skv, torch.bfloat16, seed=3), label=f"fwd_ragged{skv}")


def test_fwd_key_padding(cuda_device):
    # per-sample valid lengths incl. a sample with no valid key at all on this shard
    check(*run_case(cuda_device, 3, 4, 2, 128, 1024, torch.bfloat16, seed=5, kv_valid=[1024, 300, 0]), label="fwd_keypad")


def test_fwd_travelling_merge(cuda_device):
    """Two shards merged through the travelling accumulator == attention over the concatenation."""
    from lv_xattn_b200 import ops
    B, Hq, Hkv, Sq, Skv = 1, 8, 2, 128, 2048
    q, k, v, _ = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 7, torch.bfloat16)
    o_ref, lse_ref = orc.attention_fwd(q, k, v, SCALE)
    d = cuda_device
    qd = q.to(d)
    o1, l1 = ops.fwd_block(qd, k[:, :, :1024].to(d), v[:, :, :1024].to(d), SCALE, final=False)
    o2, l2 = ops.fwd_block(qd, k[:, :, 1024:].to(d), v[:, :, 1024:].to(d), SCALE, o_in=o1, lse_in=l1, final=True)
    torch.cuda.synchronize()
    check(o2.float().cpu(), l2.cpu().view(B, Hq, Sq), o_ref, lse_ref, label="fwd_travelling")
