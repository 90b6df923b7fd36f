"""Parity criteria shared by the GPU tests.

The stated bars are absolute (16-bit: O/dQ/dK/dV max-abs <= 2e-2, lse <= 1e-3; fp32: 1e-4). At long key
sequences the tensors themselves are far smaller than 2e-2 (softmax averages over many keys), so an absolute
bar alone cannot fail there. Every comparison therefore also requires, per tensor,
    ||got - ref||_F / ||ref||_F <= rel_fro (1e-2)     and     max|got - ref| <= rel_max * max|ref| (2e-2).
For bf16 results the floor of the first is the output rounding itself (2^-9 / sqrt(3) ~ 1.1e-3); the bars below
leave a factor of a few over what the kernels measure, and an all-zero or half-scaled tensor fails them at any size.
"""
import json
import os

import torch

# name -> (abs, rel_fro, rel_max) for 16-bit inputs. Measured over the whole GPU suite on a B200: relative Frobenius
# error at most 2.9e-3 (O 2.6e-3, dQ 2.9e-3, dK 2.9e-3, dV 2.4e-3), max error / max|ref| at most 5.3e-3; the bars are
# about 3x that.
BF16 = {"o": (2e-2, 1e-2, 2e-2), "dq": (2e-2, 1e-2, 2e-2), "dk": (2e-2, 1e-2, 2e-2), "dv": (2e-2, 1e-2, 2e-2)}
LSE_ABS_16 = 1e-3
FP32_ABS = 1e-4
FP32_REL_FRO = 1e-4

MEASURED = []      # (label, name, max_abs, rel_fro, rel_max) of every comparison of the session


def errors(got: torch.Tensor, ref: torch.Tensor):
    """(max-abs error, Frobenius error relative to the reference, max-abs error relative to max|ref|)."""
    g, r = got.double(), ref.double()
    d = g - r
    max_abs = d.abs().max().item() if d.numel() else 0.0
    rn = r.norm().item()
    rm = r.abs().max().item() if r.numel() else 0.0
    rel_fro = d.norm().item() / rn if rn > 0 else (0.0 if d.norm().item() == 0 else float("inf"))
    rel_max = max_abs / rm if rm > 0 else (0.0 if max_abs == 0 else float("inf"))
    return max_abs, rel_fro, rel_max


def assert_close(got, ref, name, label="", abs_tol=2e-2, rel_fro=1e-2, rel_max=2e-2):
    """got vs ref under the three criteria; `name` is o/dq/dk/dv, `label` identifies the case in the message."""
    assert got.shape == ref.shape, f"{label} {name}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got.float()).all(), f"{label} {name}: non-finite values"
    ma, rf, rm = errors(got, ref)
    MEASURED.append((label, name, ma, rf, rm))
    ref_max = ref.abs().max().item() if ref.numel() else 0.0
    assert ma <= abs_tol, f"{label} {name}: max-abs err {ma:.3e} > {abs_tol} (max|ref| {ref_max:.3e})"
    assert rf <= rel_fro, f"{label} {name}: relative Frobenius err {rf:.3e} > {rel_fro} (max|ref| {ref_max:.3e})"
    assert rm <= rel_max, f"{label} {name}: max err / max|ref| = {rm:.3e} > {rel_max} (max|ref| {ref_max:.3e})"


def assert_lse_close(got, ref, label="", abs_tol=LSE_ABS_16):
    """lse: the same rows are -inf on both sides, and the finite ones agree to abs_tol (lse is O(10), so the
    absolute bar is already a relative one of 1e-4)."""
    fin = torch.isfinite(ref)
    assert torch.equal(torch.isfinite(got), fin), f"{label} lse: -inf rows differ"
    if fin.any():
        e = (got[fin].double() - ref[fin].double()).abs().max().item()
        MEASURED.append((label, "lse", e, 0.0, 0.0))
        assert e <= abs_tol, f"{label} lse: max-abs err {e:.3e} > {abs_tol}"


def assert_grads_16bit(got, ref, label=""):
    """(dq, dk, dv) of a 16-bit case against the fp32 oracle."""
    for name, g, r in zip(("dq", "dk", "dv"), got, ref):
        a, f, m = BF16[name]
        assert_close(g.float().cpu(), r.float().cpu(), name, label, a, f, m)


def assert_fp32(got, ref, name, label=""):
    assert_close(got, ref, name, label, FP32_ABS, FP32_REL_FRO, 1e-3)


def dump_measured():
    """Writes what every comparison measured to $LVX_PARITY_LOG (JSON lines), when that is set."""
    path = os.environ.get("LVX_PARITY_LOG")
    if not path or not MEASURED:
        return
    with open(path, "a") as f:
        for label, name, ma, rf, rm in MEASURED:
            f.write(json.dumps({"case": label, "tensor": name, "max_abs": ma, "rel_fro": rf, "rel_max": rm}) + "\n")
