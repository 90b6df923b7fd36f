"""lvx_fwd_block_static: the forward block for callers that must not allocate device memory at call time
(fixed memory budget, no allocator call or device synchronisation allowed on their path). It keeps its
split-KV scratch in a 32 MiB area inside the library, so the only buffers involved are the caller's inputs
and outputs. The file sorts last so that a stop-at-first-failure run has already exercised everything else.

Called through the C ABI, twice in a row with different inputs (the scratch is shared and keeps the previous
call's contents), and compared with the workspace-based entry points on the same inputs within the 16-bit
tolerances used throughout the tests (O 2e-2 max-abs, lse 1e-3); also against the CPU oracle."""
import ctypes
import math

import pytest
import torch

import _parity
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
SCALE = 1.0 / math.sqrt(128.0)


def call_static(q, k, v, kv_valid=None):
    from lv_xattn_b200 import _lib, ops
    lib = _lib.load()
    B, Hq, Sq, D = q.shape
    shp = ops.shape_of(q, k)
    o = torch.empty_like(q)
    lse = torch.empty(B * Hq, Sq, dtype=torch.float32, device=q.device)
    rc = lib.lvx_fwd_block_static(ctypes.byref(shp), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kv_valid),
                                  ctypes.c_float(SCALE), _lib.ptr(o), _lib.ptr(lse), _lib.stream_ptr())
    return rc, o, lse


@pytest.mark.parametrize("shape", [
    (1, 8, 2, 128, 2048),       # fits with the regular split plan
    (1, 32, 8, 1024, 8192),     # regular plan would need > 32 MiB of partials: splits are lowered
])
def test_static_matches_workspace_entry_point_twice(cuda_device, shape):
    from lv_xattn_b200 import _lib, ops
    B, Hq, Hkv, Sq, Skv = shape
    for seed in (41, 42):       # two calls in a row, different data
        q, k, v, _ = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, seed, torch.bfloat16)
        qd, kd, vd = (t.to(cuda_device) for t in (q, k, v))
        rc, o, lse = call_static(qd, kd, vd)
        assert rc == 0, _lib.load().lvx_last_error()
        o_ws, lse_ws = ops.fwd_block(qd, kd, vd, SCALE)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        _parity.assert_close(o.float(), o_ws.float(), "o", f"static_vs_ws{shape}", *_parity.BF16["o"])
        assert (lse - lse_ws).abs().max().item() <= 1e-3
        o_ref, lse_ref = orc.attention_fwd(q, k, v, SCALE)
        _parity.assert_close(o.float().cpu(), o_ref, "o", f"static{shape}", *_parity.BF16["o"])
        _parity.assert_lse_close(lse.cpu().view(B, Hq, Sq), lse_ref, f"static{shape}")


def test_static_key_padding(cuda_device):
    from lv_xattn_b200 import _lib
    B, Hq, Hkv, Sq, Skv = 2, 4, 2, 64, 1024
    q, k, v, _ = orc.make_inputs(B, Hq, Hkv, Sq, Skv, 128, 43, torch.float16)
    valid = [700, 0]
    kvl = torch.tensor(valid, dtype=torch.int32, device=cuda_device)
    rc, o, lse = call_static(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), kvl)
    torch.cuda.synchronize()
    assert rc == 0, _lib.load().lvx_last_error()
    o_ref, lse_ref = orc.attention_fwd(q, k, v, SCALE, valid)
    _parity.assert_lse_close(lse.cpu().view(B, Hq, Sq), lse_ref, "static_keypad")
    _parity.assert_close(o.float().cpu(), o_ref, "o", "static_keypad", *_parity.BF16["o"])


def test_static_rejects_oversized_shape(cuda_device):
    from lv_xattn_b200 import _lib
    # 32 heads x 2048 rows = 65,536 rows: unsplit partials are just over 32 MiB
    q = torch.zeros(1, 32, 2048, 128, dtype=torch.bfloat16, device=cuda_device)
    k = torch.zeros(1, 8, 256, 128, dtype=torch.bfloat16, device=cuda_device)
    rc, _, _ = call_static(q, k, k)
    assert rc == -8                      # LVX_ERR_LIMIT
    assert b"32" in _lib.load().lvx_last_error() or b"scratch" in _lib.load().lvx_last_error()
