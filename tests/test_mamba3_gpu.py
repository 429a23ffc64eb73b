"""Parity of the CUDA Mamba-3 scan (through the C ABI) with the CPU oracle."""
import json
import os

import numpy as np
import pytest
import torch

from mixlab_b200 import ops
from oracle import inputs, mamba3
from tests.util import assert_close, rel_errs

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"
ARGS = ("x", "dt_raw", "lambda_raw", "theta", "a_log", "b", "c")
GRADS = ("dx", "ddt", "dlambda", "dtheta", "da_log", "db", "dc")


def _dev(t):
    return t.to(DEV).contiguous()


def _check_grads(got, want, tol):
    """The reference's own acceptance rule (train/gpu_trainer_mamba3_test.go:374-384) is
    max-rel <= 3e-3 or max-abs <= 3e-5 per gradient family; here: relative to the family's scale."""
    for name in GRADS:
        assert_close(got[name], want[name], tol, name)


@pytest.mark.parametrize("shape", [
    (2, 8, 4, 8, 1), (2, 8, 4, 8, 2),            # the reference test's shapes
    (2, 130, 8, 8, 2), (2, 130, 8, 64, 1), (1, 130, 8, 128, 2), (1, 33, 4, 256, 1),
    (1, 70, 24, 16, 1), (2, 50, 40, 8, 2),        # several CTAs per group: partial rows added in slice order
    (2, 50, 24, 32, 2), (1, 40, 8, 8, 1),         # two / four channels per warp (d_state <= 32 / <= 16)
    (1, 40, 6, 8, 1),                             # channels of a group do not fill whole warps: one channel per warp
])
def test_per_channel_fp32(shape):
    B, T, D, N, Gr = shape
    a = inputs.mamba3_inputs(B, T, D, 1, N, G=Gr, seed=3, per_head=False)
    f = [a[k].double() for k in ARGS]
    y_ref, want = mamba3.scan_vjp(*f, a["dy"].double())
    dev = [_dev(a[k]) for k in ARGS]
    y = ops.mamba3_selective_scan(*dev)
    assert_close(y, y_ref, 1e-4, "y")
    got = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]))
    _check_grads(got, want, 1e-4)


def test_reference_golden_vectors():
    with open(os.path.join(G, "mamba3_scalar_reference.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        B, T, D, N, Gr = (c[x] for x in ("B", "T", "D", "N", "G"))
        t = lambda key, *s: _dev(torch.tensor(c[key], dtype=torch.float32).reshape(*s))
        y = ops.mamba3_selective_scan(t("x", B, T, D), t("dt_raw", B, T, D), t("lambda_raw", B, T, D),
                                      t("theta", B, T, D, N // 2), t("a_log", D, N), t("b", B, T, Gr, N),
                                      t("c", B, T, Gr, N))
        assert_close(y, torch.tensor(c["y"], dtype=torch.float64).reshape(B, T, D), 1e-4, c["name"])
    z = np.load(os.path.join(G, "mamba3_torch_scan.npz"))
    for tag in ("a", "b", "c"):
        a = {k[2:]: torch.from_numpy(z[k]) for k in z.files if k.startswith(tag + "_")}
        y = ops.mamba3_selective_scan(*(_dev(a[k].float()) for k in ARGS))
        assert_close(y, a["y"], 1e-4, f"torch_scan_{tag}")


@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
def test_per_head_layout(io):
    """Head-broadcast parameters (benchmark config 3 layout) at a reduced size."""
    B, T, H, P, N = 2, 96, 2, 8, 128
    a = inputs.mamba3_inputs(B, T, H, P, N, G=1, seed=3, io_dtype=io, per_head=True)
    full = inputs.mamba3_expand_per_head(a)
    y_ref, want = mamba3.scan_vjp(*(full[k].double() for k in ARGS), a["dy"].double())
    # fold per-channel reference gradients back to per-head
    want = dict(want)
    want["ddt"] = want["ddt"].reshape(B, T, H, P).sum(-1)
    want["dlambda"] = want["dlambda"].reshape(B, T, H, P).sum(-1)
    want["dtheta"] = want["dtheta"].reshape(B, T, H, P, N // 2).sum((-1, -2))
    want["da_log"] = want["da_log"].reshape(H, P, N).sum((-1, -2))
    dev = [_dev(a[k]) for k in ARGS]
    tol = 1e-4 if io == torch.float32 else 2e-2
    y = ops.mamba3_selective_scan(*dev, nheads=H)
    assert_close(y, y_ref, tol, "y")
    got = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]), nheads=H)
    _check_grads(got, want, tol)


def test_long_sequence_phase_stability():
    """T=2048: the wrapped fp32 angle must not drift against the float64 oracle."""
    B, T, D, N = 1, 2048, 4, 16
    a = inputs.mamba3_inputs(B, T, D, 1, N, G=1, seed=9, per_head=False)
    y_ref = mamba3.scan_forward(*(a[k].double() for k in ARGS))
    y = ops.mamba3_selective_scan(*(_dev(a[k]) for k in ARGS))
    e2, ei = rel_errs(y, y_ref)
    assert e2 < 1e-4 and ei < 1e-4, (e2, ei)


@pytest.mark.parametrize("cfg", [
    # B, T, nheads, headdim, N, G, io
    (2, 50, 2, 16, 128, 1, torch.float32), (1, 97, 4, 16, 64, 2, torch.float32),
    (1, 40, 2, 64, 128, 1, torch.float32), (2, 64, 2, 32, 128, 2, torch.bfloat16),
    (1, 33, 1, 64, 128, 1, torch.bfloat16),
    (1, 520, 8, 64, 128, 2, torch.float32),   # many windows, eight heads in two groups
])
def test_head_cta_kernels(cfg):
    """CTA-per-head kernels (head-broadcast layout): forward and all gradients against the float64 oracle
    and against the warp-per-channel kernels."""
    from mixlab_b200 import _lib
    B, T, H, P, N, Gr, io = cfg
    a = inputs.mamba3_inputs(B, T, H, P, N, G=Gr, seed=4, io_dtype=io, per_head=True)
    full = inputs.mamba3_expand_per_head(a)
    y_ref, want = mamba3.scan_vjp(*(full[k].double() for k in ARGS), a["dy"].double())
    want = dict(want)
    want["ddt"] = want["ddt"].reshape(B, T, H, P).sum(-1)
    want["dlambda"] = want["dlambda"].reshape(B, T, H, P).sum(-1)
    want["dtheta"] = want["dtheta"].reshape(B, T, H, P, N // 2).sum((-1, -2))
    want["da_log"] = want["da_log"].reshape(H, P, N).sum((-1, -2))
    dev = [_dev(a[k]) for k in ARGS]
    tol = 1e-4 if io == torch.float32 else 2e-2
    REC = _lib.MXB_MAMBA3_RECURRENT_KERNELS  # keep the chunked tensor-core kernels out of this test
    y = ops.mamba3_selective_scan(*dev, nheads=H, flags=REC)
    assert_close(y, y_ref, tol, "y")
    y_ch = ops.mamba3_selective_scan(*dev, nheads=H, flags=_lib.MXB_MAMBA3_CHANNEL_KERNELS)
    assert_close(y, y_ch.double(), tol, "y vs channel kernel")
    got = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]), nheads=H, flags=REC)
    _check_grads(got, want, tol)
    # the shares of a head's CTAs and warps are added in a fixed order (no floating-point atomics): a second run agrees
    # in every bit
    got = {k: v.clone() for k, v in got.items()}
    again = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]), nheads=H, flags=REC)
    for name in GRADS:
        assert torch.equal(got[name], again[name]), name


@pytest.mark.parametrize("cfg", [(1, 64, 1, 1), (2, 200, 2, 1), (1, 330, 4, 2), (1, 1, 1, 1)])
def test_chunked_tensor_core_kernels(cfg):
    """Chunked dual form on tensor cores (head dim 64, d_state 128, bf16 I/O): forward and all gradients against
    the float64 oracle on the bf16-rounded inputs (2e-2), and against the recurrent kernels."""
    from mixlab_b200 import _lib
    B, T, H, Gr = cfg
    P, N = 64, 128
    a = inputs.mamba3_inputs(B, T, H, P, N, G=Gr, seed=6, io_dtype=torch.bfloat16, per_head=True)
    full = inputs.mamba3_expand_per_head(a)
    y_ref, want = mamba3.scan_vjp(*(full[k].double() for k in ARGS), a["dy"].double())
    want = dict(want)
    want["ddt"] = want["ddt"].reshape(B, T, H, P).sum(-1)
    want["dlambda"] = want["dlambda"].reshape(B, T, H, P).sum(-1)
    want["dtheta"] = want["dtheta"].reshape(B, T, H, P, N // 2).sum((-1, -2))
    want["da_log"] = want["da_log"].reshape(H, P, N).sum((-1, -2))
    dev = [_dev(a[k]) for k in ARGS]
    y = ops.mamba3_selective_scan(*dev, nheads=H)
    assert_close(y, y_ref, 2e-2, "y")
    y_rec = ops.mamba3_selective_scan(*dev, nheads=H, flags=_lib.MXB_MAMBA3_RECURRENT_KERNELS)
    assert_close(y, y_rec.double(), 2e-2, "y vs recurrent kernels")
    got = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]), nheads=H)
    errs = {}
    for name in GRADS:
        if want[name].abs().max().item() < 1e-9:
            # e.g. T = 1: the output does not depend on the angle, the exact gradient is 0 - compare absolutely,
            # against the scale of the dt gradient
            assert got[name].abs().max().item() <= 2e-2 * want["ddt"].abs().max().item(), name
            continue
        try:
            errs[name] = assert_close(got[name], want[name], 2e-2, name)
        except AssertionError as e:
            errs[name] = str(e)[:200]
    assert all(not isinstance(v, str) for v in errs.values()), errs


@pytest.mark.parametrize("cfg", [(2, 200, 2, 1), (1, 330, 4, 2)])
def test_chunked_backward_from_saved_forward(cfg):
    """Forward with save_for_backward + backward with use_saved == backward with its own recompute, bit for bit
    (the same kernels run on the same chunk states)."""
    B, T, H, Gr = cfg
    a = inputs.mamba3_inputs(B, T, H, 64, 128, G=Gr, seed=8, io_dtype=torch.bfloat16, per_head=True)
    dev = [_dev(a[k]) for k in ARGS]
    dy = _dev(a["dy"])
    want = ops.mamba3_selective_scan_backward(*dev, dy, nheads=H)
    y0 = ops.mamba3_selective_scan(*dev, nheads=H)
    y = ops.mamba3_selective_scan(*dev, nheads=H, save_for_backward=True)
    got = ops.mamba3_selective_scan_backward(*dev, dy, nheads=H, use_saved=True)
    assert torch.equal(y, y0)
    for name in GRADS:
        assert torch.equal(got[name], want[name]), name


def test_chunked_kernels_without_tma_match():
    """The cp.async staging path (MXB_MAMBA3_NO_TMA) gives the same results as the copy-engine path, bit for bit
    (same arithmetic on the same tiles, only the shared-memory layout of the operands differs)."""
    from mixlab_b200 import _lib
    B, T, H, Gr = 2, 200, 2, 1
    a = inputs.mamba3_inputs(B, T, H, 64, 128, G=Gr, seed=9, io_dtype=torch.bfloat16, per_head=True)
    dev = [_dev(a[k]) for k in ARGS]
    dy = _dev(a["dy"])
    y = ops.mamba3_selective_scan(*dev, nheads=H)
    y2 = ops.mamba3_selective_scan(*dev, nheads=H, flags=_lib.MXB_MAMBA3_NO_TMA)
    assert torch.equal(y, y2)
    g1 = ops.mamba3_selective_scan_backward(*dev, dy, nheads=H)
    g2 = ops.mamba3_selective_scan_backward(*dev, dy, nheads=H, flags=_lib.MXB_MAMBA3_NO_TMA)
    for name in GRADS:
        assert torch.equal(g1[name], g2[name]), name


@pytest.mark.parametrize("form", ["serial", "windows"])
@pytest.mark.parametrize("case", [(2, 1024, 128, 16, 4, False, torch.float32),   # the shape the reference publishes
                                  (2, 100, 48, 8, 1, False, torch.bfloat16),
                                  (1, 70, 8, 256, 1, False, torch.float32),     # four state pairs per lane
                                  (2, 100, 32, 16, 2, True, torch.float32)])
def test_channel_kernels_repeat_bit_for_bit(case, form):
    """The warp-per-channel kernels, as one walk per (batch, channel) and window-parallel, add over channels, windows
    and the batch in a fixed order (no floating-point atomics): two runs on the same inputs agree in every bit, and
    the result matches the oracle."""
    from mixlab_b200 import _lib
    B, T, D, N, Gr, per_head, io = case
    nheads = D // 8 if per_head else 1
    a = inputs.mamba3_inputs(B, T, nheads if per_head else D, 8 if per_head else 1, N, G=Gr, seed=9,
                             io_dtype=io, per_head=per_head)
    dev = [_dev(a[k]) for k in ARGS]
    flags = _lib.MXB_MAMBA3_SERIAL_WALK if form == "serial" else _lib.MXB_MAMBA3_WINDOW_PARALLEL
    kw = dict(flags=flags)
    if per_head:
        kw = dict(nheads=nheads, flags=flags | _lib.MXB_MAMBA3_CHANNEL_KERNELS)
    first = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]), **kw)
    first = {k: v.clone() for k, v in first.items()}
    y = ops.mamba3_selective_scan(*dev, **kw)  # something else through the workspace in between
    second = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]), **kw)
    for name in GRADS:
        assert torch.equal(first[name], second[name]), name
    e = inputs.mamba3_expand_per_head(a) if per_head else a
    f = [e[k].double() for k in ARGS]
    y_ref, want = mamba3.scan_vjp(*f, a["dy"].double())
    if per_head:  # gradients of broadcast parameters are the sums over what they were broadcast to
        P = 8
        want = dict(want)
        want["ddt"] = want["ddt"].reshape(B, T, nheads, P).sum(-1)
        want["dlambda"] = want["dlambda"].reshape(B, T, nheads, P).sum(-1)
        want["dtheta"] = want["dtheta"].reshape(B, T, nheads, P, N // 2).sum((-1, -2))
        want["da_log"] = want["da_log"].reshape(nheads, P, N).sum((-1, -2))
    tol = 1e-4 if io == torch.float32 else 2e-2
    assert_close(y, y_ref, tol, "y")
    _check_grads(second, want, tol)


@pytest.mark.parametrize("shape", [(2, 130, 8, 8, 2), (1, 17, 4, 64, 1), (1, 16, 4, 8, 1), (2, 5, 4, 8, 2)])
def test_window_parallel_matches_serial_walk(shape):
    """Both forms of the channel kernels compute the same recurrence: windows that end inside the sequence, a last
    window of one step, a single window."""
    from mixlab_b200 import _lib
    B, T, D, N, Gr = shape
    a = inputs.mamba3_inputs(B, T, D, 1, N, G=Gr, seed=21, per_head=False)
    dev = [_dev(a[k]) for k in ARGS]
    ys = ops.mamba3_selective_scan(*dev, flags=_lib.MXB_MAMBA3_SERIAL_WALK)
    yw = ops.mamba3_selective_scan(*dev, flags=_lib.MXB_MAMBA3_WINDOW_PARALLEL)
    assert_close(yw, ys.double(), 1e-5, "y")
    gs = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]), flags=_lib.MXB_MAMBA3_SERIAL_WALK)
    gw = ops.mamba3_selective_scan_backward(*dev, _dev(a["dy"]), flags=_lib.MXB_MAMBA3_WINDOW_PARALLEL)
    for name in GRADS:
        assert_close(gw[name], gs[name].double(), 1e-5, name)
