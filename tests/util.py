"""Shared helpers for the parity tests."""
import torch


def rel_errs(got: torch.Tensor, ref: torch.Tensor):
    """(||got-ref||_2 / ||ref||_2 , max|got-ref| / max|ref|) in float64."""
    g = got.detach().double().cpu().flatten()
    r = ref.detach().double().cpu().flatten()
    den2 = max(r.norm().item(), 1e-30)
    deni = max(r.abs().max().item(), 1e-30) if r.numel() else 1.0
    if r.numel() == 0:
        return 0.0, 0.0
    return (g - r).norm().item() / den2, (g - r).abs().max().item() / deni


def assert_close(got, ref, tol, name=""):
    assert got.shape == ref.shape, (name, tuple(got.shape), tuple(ref.shape))
    assert torch.isfinite(got.float()).all(), f"{name}: non-finite values"
    e2, ei = rel_errs(got, ref)
    assert e2 <= tol and ei <= tol, f"{name}: rel-l2 {e2:.3e} rel-max {ei:.3e} > {tol:g}"
    return e2, ei
