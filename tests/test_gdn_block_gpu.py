"""Element-wise stages of the gated_deltanet block (conv + SiLU + L2-norm, gate/beta, output norm x gate) through
the C ABI against the CPU oracle (oracle/gdn_block.py, pinned to the reference's scalar helpers) and against the
committed golden vectors; forward and every gradient."""
import json
import os

import pytest
import torch

from mixlab_b200 import ops
from oracle import gdn_block
from util import assert_close

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


def _inputs(B, T, H, Dk, Dv, seed, io):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    d = dict(q_proj=r(B, T, H * Dk).to(io), k_proj=r(B, T, H * Dk).to(io), v_proj=r(B, T, H * Dv).to(io),
             conv_q=0.4 * r(4, H * Dk), conv_k=0.4 * r(4, H * Dk), conv_v=0.4 * r(4, H * Dv),
             a_raw=r(B, T, H), b_raw=r(B, T, H), a_log=0.5 * r(H), dt_bias=0.3 * r(H),
             o=r(B, T, H, Dv).to(io), z=r(B, T, H * Dv).to(io), o_norm=1.0 + 0.2 * r(Dv),
             dq=r(B, T, H, Dk).to(io), dk=r(B, T, H, Dk).to(io), dv=r(B, T, H, Dv).to(io),
             dbeta=r(B, T, H), dgate=r(B, T, H), dy=r(B, T, H * Dv).to(io))
    return d


PRE = ("q_proj", "k_proj", "v_proj", "conv_q", "conv_k", "conv_v", "a_raw", "b_raw", "a_log", "dt_bias")


def _oracle_pre(d, H, Dk, Dv, gate_is_log):
    x = {k: d[k].double().requires_grad_(True) for k in PRE}
    outs = gdn_block.block_pre(*(x[k] for k in PRE), H, Dk, Dv, gate_is_log=gate_is_log)
    loss = sum((o * d[n].double().reshape(o.shape)).sum() for o, n in zip(outs, ("dq", "dk", "dv", "dbeta", "dgate")))
    grads = torch.autograd.grad(loss, [x[k] for k in PRE])
    return outs, dict(zip(PRE, grads))


@pytest.mark.parametrize("cfg", [(2, 70, 2, 16, 24), (1, 3, 1, 8, 8), (1, 200, 2, 128, 128), (2, 65, 3, 64, 128)])
@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("gate_is_log", [False, True])
def test_block_pre_forward_and_gradients(cfg, io, gate_is_log):
    B, T, H, Dk, Dv = cfg
    d = _inputs(B, T, H, Dk, Dv, 11, io)
    tol = 1e-4 if io == torch.float32 else 2e-2
    (q, k, v, beta, gate), want = _oracle_pre(d, H, Dk, Dv, gate_is_log)
    dev = {n: t.to(DEV) for n, t in d.items()}
    got = ops.gdn_block_pre(*(dev[n] for n in PRE), H, Dk, Dv, gate_is_log=gate_is_log)
    for g_, w_, name in zip(got, (q, k, v, beta, gate), ("q", "k", "v", "beta", "gate")):
        assert_close(g_, w_.detach(), tol, name)
    gr = ops.gdn_block_pre_backward(*(dev[n] for n in PRE), H, Dk, Dv, dev["dq"], dev["dk"], dev["dv"], dev["dbeta"],
                                    dev["dgate"], gate_is_log=gate_is_log)
    names = dict(q_proj="dq_proj", k_proj="dk_proj", v_proj="dv_proj", conv_q="dconv_q", conv_k="dconv_k",
                 conv_v="dconv_v", a_raw="da_raw", b_raw="db_raw", a_log="da_log", dt_bias="ddt_bias")
    for src, name in names.items():
        assert_close(gr[name], want[src], tol, name)


@pytest.mark.parametrize("cfg", [(2, 70, 2, 24), (1, 3, 1, 8), (1, 300, 4, 128)])
@pytest.mark.parametrize("io", [torch.float32, torch.bfloat16])
def test_block_post_forward_and_gradients(cfg, io):
    B, T, H, Dv = cfg
    d = _inputs(B, T, H, 8, Dv, 12, io)
    tol = 1e-4 if io == torch.float32 else 2e-2
    x = {k: d[k].double().requires_grad_(True) for k in ("o", "z", "o_norm")}
    y = gdn_block.block_post(x["o"], x["z"], x["o_norm"])
    go, gz, gw = torch.autograd.grad((y * d["dy"].double()).sum(), [x["o"], x["z"], x["o_norm"]])
    dev = {n: t.to(DEV) for n, t in d.items()}
    assert_close(ops.gdn_block_post(dev["o"], dev["z"], dev["o_norm"]), y.detach(), tol, "y")
    gr = ops.gdn_block_post_backward(dev["o"], dev["z"], dev["o_norm"], dev["dy"])
    assert_close(gr["do"], go, tol, "do")
    assert_close(gr["dz"], gz, tol, "dz")
    assert_close(gr["do_norm"], gw, tol, "do_norm")


def test_block_stages_golden_vectors():
    """The vectors made by the reference's own scalar helpers (fp32 I/O; only the case with Dk, Dv multiples of 8)."""
    data = json.load(open(os.path.join(G, "gdn_block_stages.json")))
    ran = 0
    for c in data["cases"]:
        B, T, H, Dk, Dv = (c[k] for k in ("B", "T", "H", "Dk", "Dv"))
        if Dk % 8 or Dv % 8:
            continue
        t = lambda name, *shape: torch.tensor(c[name], dtype=torch.float32).reshape(*shape).to(DEV)
        q, k, v, beta, gate = ops.gdn_block_pre(
            t("q_proj", B, T, H * Dk), t("k_proj", B, T, H * Dk), t("v_proj", B, T, H * Dv), t("conv_q", 4, H * Dk),
            t("conv_k", 4, H * Dk), t("conv_v", 4, H * Dv), t("a_raw", B, T, H), t("b_raw", B, T, H), t("a_log", H),
            t("dt_bias", H), H, Dk, Dv)
        for got, name, shape in ((q, "q", (B, T, H, Dk)), (k, "k", (B, T, H, Dk)), (v, "v", (B, T, H, Dv)),
                                 (beta, "beta", (B, T, H)), (gate, "gate", (B, T, H))):
            assert_close(got, torch.tensor(c[name], dtype=torch.float64).reshape(*shape), 1e-4, name)
        y = ops.gdn_block_post(t("o", B, T, H, Dv), t("z", B, T, H * Dv), t("o_norm", Dv))
        assert_close(y, torch.tensor(c["y"], dtype=torch.float64).reshape(B, T, H * Dv), 1e-4, "y")
        ran += 1
    assert ran >= 2
