"""The CPU oracle against the reference's own golden vectors (tests/golden/)."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import gdn, mamba3

G = os.path.join(os.path.dirname(__file__), "golden")
F64 = torch.float64


def _t(a, *shape):
    return torch.tensor(a, dtype=F64).reshape(*shape)


def _gdn_cases():
    with open(os.path.join(G, "gdn_scalar_reference.json")) as f:
        return json.load(f)["cases"]


@pytest.mark.parametrize("case", _gdn_cases(), ids=lambda c: c["name"])
@pytest.mark.parametrize("chunk", [0, 4, 64])
def test_gdn_scalar_reference(case, chunk):
    B, T, H, K, V = (case[x] for x in ("B", "T", "H", "Dk", "Dv"))
    q, k = _t(case["q"], B, T, H, K), _t(case["k"], B, T, H, K)
    v = _t(case["v"], B, T, H, V)
    beta, gate = _t(case["beta"], B, T, H), _t(case["gate"], B, T, H)
    want = _t(case["out"], B, T, H, V)
    got, _ = gdn.scan_chunked(q, k, v, beta, gate, chunk)
    assert torch.max(torch.abs(got - want)).item() < 1e-11


@pytest.mark.parametrize("chunk", [0, 64, 16])
def test_gdn_torch_recurrence(chunk):
    z = np.load(os.path.join(G, "gdn_torch_recurrence.npz"))
    a = {k: torch.from_numpy(z[k]) for k in z.files}
    got, _ = gdn.scan_chunked(a["q"], a["k"], a["v"], a["beta"], a["gate"], chunk)
    assert torch.max(torch.abs(got - a["out"])).item() < 1e-11


def test_gdn_go_test_chunked_matches_naive():
    """gpu/gated_delta_scan_test.go:174-263: chunk 64 == naive on the closed-form
    inputs, output tol 1e-4, gradient tol 1e-6 (here in float64, far tighter)."""
    z = np.load(os.path.join(G, "gdn_go_test_inputs.npz"))
    a = {k: torch.from_numpy(z[k]) for k in z.files}
    o_n, s_n = gdn.scan_naive(a["q"], a["k"], a["v"], a["beta"], a["gate"])
    o_c, s_c = gdn.scan_chunked(a["q"], a["k"], a["v"], a["beta"], a["gate"], 64)
    assert torch.max(torch.abs(o_n - o_c)).item() < 1e-12
    assert torch.max(torch.abs(s_n - s_c)).item() < 1e-12
    # mean-square loss gradients as TrainerComputeMeanSquareGrads does
    d_out = 2.0 * o_n / o_n.numel()
    gn = gdn.scan_grads(a["q"], a["k"], a["v"], a["beta"], a["gate"], d_out, chunk_size=0)
    gc = gdn.scan_grads(a["q"], a["k"], a["v"], a["beta"], a["gate"], d_out, chunk_size=64)
    for name in ("dq", "dk", "dv", "dbeta", "dgate"):
        assert torch.max(torch.abs(gn[name] - gc[name])).item() < 1e-12, name


def test_gdn_fp32_chunked_vs_naive_reference_tolerance():
    """Same test in float32, at the reference's own tolerance (1e-4)."""
    z = np.load(os.path.join(G, "gdn_go_test_inputs.npz"))
    a = {k: torch.from_numpy(z[k]).float() for k in z.files}
    o_n, _ = gdn.scan_naive(a["q"], a["k"], a["v"], a["beta"], a["gate"])
    o_c, _ = gdn.scan_chunked(a["q"], a["k"], a["v"], a["beta"], a["gate"], 64)
    assert torch.max(torch.abs(o_n - o_c)).item() < 1e-4


def test_solve_strictly_lower_and_vjp():
    g = torch.Generator().manual_seed(0)
    raw = torch.tril(torch.randn(3, 16, 16, generator=g, dtype=F64) * 0.3, -1)
    raw.requires_grad_(True)
    X = gdn.solve_strictly_lower(raw)
    eye = torch.eye(16, dtype=F64)
    assert torch.max(torch.abs(X - torch.linalg.inv(eye - raw))).item() < 1e-12
    cot = torch.randn(3, 16, 16, generator=g, dtype=F64)
    (auto,) = torch.autograd.grad((X * cot).sum(), raw)
    want = gdn.solve_strictly_lower_vjp(X.detach(), cot)
    assert torch.max(torch.abs(torch.tril(auto, -1) - want)).item() < 1e-12


def test_gdn_decode_step_is_scan_body():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(2, 5, 3, 4, generator=g, dtype=F64)
    k = torch.randn(2, 5, 3, 4, generator=g, dtype=F64)
    v = torch.randn(2, 5, 3, 6, generator=g, dtype=F64)
    beta = torch.rand(2, 5, 3, generator=g, dtype=F64)
    gate = torch.rand(2, 5, 3, generator=g, dtype=F64)
    out, S = gdn.scan_naive(q, k, v, beta, gate)
    st = torch.zeros(2, 3, 4, 6, dtype=F64)
    for t in range(5):
        o, st = gdn.decode_step(st, q[:, t], k[:, t], v[:, t], beta[:, t], gate[:, t])
        assert torch.equal(o, out[:, t])
    assert torch.equal(st, S)


def test_mamba3_scalar_reference():
    with open(os.path.join(G, "mamba3_scalar_reference.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        B, T, D, N, Gr = (c[x] for x in ("B", "T", "D", "N", "G"))
        y = mamba3.scan_forward(_t(c["x"], B, T, D), _t(c["dt_raw"], B, T, D), _t(c["lambda_raw"], B, T, D),
                                _t(c["theta"], B, T, D, N // 2), _t(c["a_log"], D, N),
                                _t(c["b"], B, T, Gr, N), _t(c["c"], B, T, Gr, N))
        assert torch.max(torch.abs(y - _t(c["y"], B, T, D))).item() < 1e-12


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_mamba3_torch_scan_and_vjp(tag):
    z = np.load(os.path.join(G, "mamba3_torch_scan.npz"))
    a = {k[2:]: torch.from_numpy(z[k]) for k in z.files if k.startswith(tag + "_")}
    args = (a["x"], a["dt_raw"], a["lambda_raw"], a["theta"], a["a_log"], a["b"], a["c"])
    y = mamba3.scan_forward(*args)
    assert torch.max(torch.abs(y - a["y"])).item() < 1e-11
    # closed-form VJP (restated from the reference's float64 Go oracle) == autograd
    g = torch.Generator().manual_seed(5)
    dy = torch.randn(y.shape, generator=g, dtype=F64)
    y2, closed = mamba3.scan_vjp(*args, dy)
    _, auto = mamba3.scan_grads_autograd(*args, dy)
    assert torch.max(torch.abs(y2 - y)).item() < 1e-12
    for name, gr in auto.items():
        err = torch.max(torch.abs(closed[name] - gr)).item()
        scale = max(1.0, torch.max(torch.abs(gr)).item())
        assert err / scale < 1e-10, (name, err)


def test_gdn_block_stages_match_reference_helpers():
    """oracle.gdn_block against vectors from the reference's own scalar block helpers."""
    from oracle import gdn_block
    data = json.load(open(os.path.join(G, "gdn_block_stages.json")))
    for c in data["cases"]:
        B, T, H, Dk, Dv = (c[k] for k in ("B", "T", "H", "Dk", "Dv"))
        t = lambda name, *shape: torch.tensor(c[name], dtype=torch.float64).reshape(*shape)
        q, k, v, beta, gate = gdn_block.block_pre(
            t("q_proj", B, T, H * Dk), t("k_proj", B, T, H * Dk), t("v_proj", B, T, H * Dv), t("conv_q", 4, H * Dk),
            t("conv_k", 4, H * Dk), t("conv_v", 4, H * Dv), t("a_raw", B, T, H), t("b_raw", B, T, H), t("a_log", H),
            t("dt_bias", H), H, Dk, Dv)
        for got, name, shape in ((q, "q", (B, T, H, Dk)), (k, "k", (B, T, H, Dk)), (v, "v", (B, T, H, Dv)),
                                 (beta, "beta", (B, T, H)), (gate, "gate", (B, T, H))):
            assert (got - t(name, *shape)).abs().max().item() < 1e-12, name
        y = gdn_block.block_post(t("o", B, T, H, Dv), t("z", B, T, H * Dv), t("o_norm", Dv))
        assert (y - t("y", B, T, H * Dv)).abs().max().item() < 1e-12


def test_mamba3_block_stages_match_reference_helpers():
    """oracle.mamba3_block against vectors from the reference's own scalar block helpers."""
    from oracle import mamba3_block
    data = json.load(open(os.path.join(G, "mamba3_block_stages.json")))
    for c in data["cases"]:
        B, T, D, N, Gr, K = (c[k] for k in ("B", "T", "D", "N", "G", "K"))
        t = lambda name, *shape: torch.tensor(c[name], dtype=torch.float64).reshape(*shape)
        conv = mamba3_block.depthwise_conv(t("x", B, T, D), t("conv_w", D, K))
        assert (conv - t("conv", B, T, D)).abs().max().item() < 1e-12
        b, cc = mamba3_block.bc_norm(t("b_proj", B, T, Gr * N), t("c_proj", B, T, Gr * N), t("b_scale", N), t("c_scale", N),
                                     t("b_bias", Gr * N), t("c_bias", Gr * N), Gr, N)
        assert (b - t("b", B, T, Gr, N)).abs().max().item() < 1e-12
        assert (cc - t("c", B, T, Gr, N)).abs().max().item() < 1e-12
        out = mamba3_block.post(t("y", B, T, D), t("z", B, T, D), t("post_norm", D))
        assert (out - t("out", B, T, D)).abs().max().item() < 1e-12
