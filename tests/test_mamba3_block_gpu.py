"""Element-wise stages of the canonical Mamba-3 block (depthwise conv, B/C RMSNorm + bias, post-norm x SiLU gate)
through the C ABI against the CPU oracle (oracle/mamba3_block.py, pinned to the reference's scalar helpers) and against
the committed golden vectors; forward and every gradient."""
import json
import os

import pytest
import torch

from mixlab_b200 import ops
from oracle import mamba3_block
from util import assert_close

pytestmark = pytest.mark.gpu
G_DIR = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


def _r(seed):
    g = torch.Generator().manual_seed(seed)
    return lambda *s: torch.randn(*s, generator=g)


@pytest.mark.parametrize("cfg", [(2, 37, 24, 4), (1, 3, 8, 2), (1, 130, 2048, 4), (2, 17, 72, 1), (1, 64, 1040, 3)])
@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
def test_conv_forward_and_gradients(cfg, io):
    B, T, D, K = cfg
    r = _r(21)
    x, w, dy = r(B, T, D).to(io), 0.4 * r(D, K), r(B, T, D).to(io)
    tol = 1e-4 if io == torch.float32 else 2e-2
    x64, w64 = x.double().requires_grad_(True), w.double().requires_grad_(True)
    y = mamba3_block.depthwise_conv(x64, w64)
    gx, gw = torch.autograd.grad((y * dy.double()).sum(), [x64, w64])
    assert_close(ops.mamba3_block_conv(x.to(DEV), w.to(DEV)), y.detach(), tol, "y")
    got = ops.mamba3_block_conv_backward(x.to(DEV), w.to(DEV), dy.to(DEV))
    assert_close(got["dx"], gx, tol, "dx")
    assert_close(got["dw"], gw, tol, "dw")


@pytest.mark.parametrize("cfg", [(2, 37, 2, 16), (1, 3, 1, 8), (1, 300, 1, 128), (2, 65, 3, 64)])
@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
def test_bc_norm_forward_and_gradients(cfg, io):
    B, T, Gr, N = cfg
    r = _r(22)
    bp, cp = r(B, T, Gr * N).to(io), r(B, T, Gr * N).to(io)
    bs, cs, bb, cb = 1 + 0.2 * r(N), 1 + 0.2 * r(N), 0.3 * r(Gr * N), 0.3 * r(Gr * N)
    db, dc = r(B, T, Gr, N).to(io), r(B, T, Gr, N).to(io)
    tol = 1e-4 if io == torch.float32 else 2e-2
    ins = [t.double().requires_grad_(True) for t in (bp, cp, bs, cs, bb, cb)]
    b, c = mamba3_block.bc_norm(*ins, Gr, N)
    grads = torch.autograd.grad((b * db.double()).sum() + (c * dc.double()).sum(), ins)
    dev = [t.to(DEV) for t in (bp, cp, bs, cs, bb, cb)]
    gb, gc = ops.mamba3_block_bc(*dev, Gr, N)
    assert_close(gb, b.detach(), tol, "b")
    assert_close(gc, c.detach(), tol, "c")
    got = ops.mamba3_block_bc_backward(dev[0], dev[1], dev[2], dev[3], db.to(DEV), dc.to(DEV), Gr, N)
    for name, want in zip(("db_proj", "dc_proj", "db_scale", "dc_scale", "db_bias", "dc_bias"), grads):
        assert_close(got[name], want, tol, name)


@pytest.mark.parametrize("cfg", [(2, 37, 24), (1, 3, 8), (1, 70, 2048), (2, 9, 1040)])
@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
def test_post_forward_and_gradients(cfg, io):
    B, T, D = cfg
    r = _r(23)
    y, z, wn, dout = r(B, T, D).to(io), r(B, T, D).to(io), 1 + 0.2 * r(D), r(B, T, D).to(io)
    tol = 1e-4 if io == torch.float32 else 2e-2
    ins = [t.double().requires_grad_(True) for t in (y, z, wn)]
    out = mamba3_block.post(*ins)
    gy, gz, gw = torch.autograd.grad((out * dout.double()).sum(), ins)
    assert_close(ops.mamba3_block_post(y.to(DEV), z.to(DEV), wn.to(DEV)), out.detach(), tol, "out")
    got = ops.mamba3_block_post_backward(y.to(DEV), z.to(DEV), wn.to(DEV), dout.to(DEV))
    assert_close(got["dy"], gy, tol, "dy")
    assert_close(got["dz"], gz, tol, "dz")
    assert_close(got["dpost_norm"], gw, tol, "dpost_norm")


def test_block_stages_golden_vectors():
    """The vectors made by the reference's own scalar helpers (fp32 I/O; the cases whose D and N are multiples of 8)."""
    data = json.load(open(os.path.join(G_DIR, "mamba3_block_stages.json")))
    ran = 0
    for c in data["cases"]:
        B, T, D, N, Gr, K = (c[k] for k in ("B", "T", "D", "N", "G", "K"))
        if D % 8 or N % 8:
            continue
        t = lambda name, *shape: torch.tensor(c[name], dtype=torch.float32).reshape(*shape).to(DEV)
        w = lambda name, *shape: torch.tensor(c[name], dtype=torch.float64).reshape(*shape)
        assert_close(ops.mamba3_block_conv(t("x", B, T, D), t("conv_w", D, K)), w("conv", B, T, D), 1e-4, "conv")
        b, cc = ops.mamba3_block_bc(t("b_proj", B, T, Gr * N), t("c_proj", B, T, Gr * N), t("b_scale", N), t("c_scale", N),
                                    t("b_bias", Gr * N), t("c_bias", Gr * N), Gr, N)
        assert_close(b, w("b", B, T, Gr, N), 1e-4, "b")
        assert_close(cc, w("c", B, T, Gr, N), 1e-4, "c")
        assert_close(ops.mamba3_block_post(t("y", B, T, D), t("z", B, T, D), t("post_norm", D)), w("out", B, T, D), 1e-4,
                     "out")
        ran += 1
    assert ran >= 2
