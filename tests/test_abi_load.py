"""CPU-side checks of the C ABI: the library loads, exports every symbol include/lvx.h declares, and refuses
bad arguments before touching a device."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from lv_xattn_b200 import _lib
    from lv_xattn_b200.build import build_lib
    build_lib()
    lib = _lib.load()
    header = open(os.path.join(ROOT, "include", "lvx.h")).read()
    declared = set(re.findall(r"\b(lvx_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.SYMBOLS), declared ^ set(_lib.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.lvx_version() == 1


def test_argument_validation_without_device():
    from lv_xattn_b200 import _lib
    lib = _lib.load()
    shp = _lib.LvxShape(1, 4, 3, 16, 16, 128, 0, 0)       # Hq not a multiple of Hkv
    f, b = ctypes.c_size_t(0), ctypes.c_size_t(0)
    assert lib.lvx_query_workspace(ctypes.byref(shp), ctypes.byref(f), ctypes.byref(b)) == -2
    assert b"multiple" in lib.lvx_last_error()
    shp = _lib.LvxShape(1, 4, 2, 16, 16, 64, 0, 0)        # head dim
    assert lib.lvx_query_workspace(ctypes.byref(shp), ctypes.byref(f), ctypes.byref(b)) == -2
    shp = _lib.LvxShape(1, 32, 8, 2048, 131072, 128, 0, 0)
    assert lib.lvx_query_workspace(ctypes.byref(shp), ctypes.byref(f), ctypes.byref(b)) == 0
    assert f.value > 0
    assert lib.lvx_add_cast(None, None, None, 0, 16, None) == -1   # NULL pointer


def test_python_entry_points_refuse_cpu_tensors():
    import pytest
    import torch
    import lv_xattn_b200 as lvx
    from lv_xattn_b200._lib import LvxError
    q = torch.zeros(1, 2, 16, 128, dtype=torch.bfloat16)
    with pytest.raises(LvxError):
        lvx._attn_forward(q, q, q, False, 0.1, None)
    with pytest.raises(NotImplementedError):
        lvx._attn_forward(q, q, q, True, 0.1, None)
    with pytest.raises(ValueError):
        lvx._attn_forward(q, q, q, False, 0.1, None, bias_func=lambda *a: None)     # bias_func must return a tensor
    with pytest.raises(ValueError):
        lvx._attn_forward(q, q, q, False, 0.1, None, local_bias_args=[q])           # arguments without a bias_func
    with pytest.raises(ValueError):
        lvx._attn_forward(q, q[:, :, :, :64], q, False, 0.1, None)
