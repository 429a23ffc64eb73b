"""Whole blocks composed from the library's stages, against the reference's own full-block fixtures.

gated_deltanet: projections (torch matmuls, they are plain matrix products) -> mxb_gdn_block_pre_* -> mxb_gdn_fwd/bwd
-> mxb_gdn_block_post_* -> output projection + residual, forward and every per-weight gradient against the vectors
the reference's generator writes (experiments/gated_deltanet_test/dump_fla_grad_reference.py, the fixture behind
train/gated_deltanet_fla_grad_parity_test.go:14-139, whose bound is max-abs <= 1e-3), with and without kv_share.
Mamba-3: the same for the canonical block against train/hf_templates/mamba3_mixlab.py (float64 torch autograd).
The CUDA stages are wired into torch autograd by small Function wrappers that call the backward entry points.
"""
import math
import os

import numpy as np
import pytest
import torch

from mixlab_b200 import ops

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"


def rmsnorm(x, w, eps=1e-5):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


class GdnPre(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qp, kp, vp, cq, ck, cv, a_raw, b_raw, a_log, dt_bias, H, Dk, Dv):
        ctx.save_for_backward(qp, kp, vp, cq, ck, cv, a_raw, b_raw, a_log, dt_bias)
        ctx.dims = (H, Dk, Dv)
        return ops.gdn_block_pre(qp, kp, vp, cq, ck, cv, a_raw, b_raw, a_log, dt_bias, H, Dk, Dv)

    @staticmethod
    def backward(ctx, dq, dk, dv, dbeta, dgate):
        H, Dk, Dv = ctx.dims
        g = ops.gdn_block_pre_backward(*ctx.saved_tensors, H, Dk, Dv, dq.contiguous(), dk.contiguous(), dv.contiguous(),
                                       dbeta.contiguous(), dgate.contiguous())
        return (g["dq_proj"], g["dk_proj"], g["dv_proj"], g["dconv_q"], g["dconv_k"], g["dconv_v"], g["da_raw"],
                g["db_raw"], g["da_log"], g["ddt_bias"], None, None, None)


class GdnScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, beta, gate, chunk):
        ctx.save_for_backward(q, k, v, beta, gate)
        ctx.chunk = chunk
        return ops.gated_delta_scan(q, k, v, beta, gate, chunk)

    @staticmethod
    def backward(ctx, d_out):
        g = ops.gated_delta_scan_backward(*ctx.saved_tensors, d_out.contiguous(), ctx.chunk)
        return g["dq"], g["dk"], g["dv"], g["dbeta"], g["dgate"], None


class GdnPost(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, z, o_norm):
        ctx.save_for_backward(o, z, o_norm)
        return ops.gdn_block_post(o, z, o_norm)

    @staticmethod
    def backward(ctx, dy):
        g = ops.gdn_block_post_backward(*ctx.saved_tensors, dy.contiguous())
        return g["do"], g["dz"], g["do_norm"]


def _oracle_stages():
    from oracle import gdn, gdn_block
    return (gdn_block.block_pre, lambda q, k, v, beta, gate, chunk: gdn.scan_chunked(q, k, v, beta, gate, chunk or 64)[0],
            gdn_block.block_post)


def _cuda_stages():
    c = lambda t: t.contiguous()
    return (lambda qp, kp, vp, cq, ck, cv, a, b, al, db, H, Dk, Dv: GdnPre.apply(c(qp), c(kp), c(vp), cq, ck, cv, c(a), c(b), al,
                                                                               db, H, Dk, Dv),
            GdnScan.apply, lambda o, z, n: GdnPost.apply(o, c(z), n))


def gdn_block_forward(x, w, H, Dk, Dv, kv_share, chunk, stages=None):
    """emitGatedDeltaNetIRWithScales (arch/blocks_gated_deltanet.go:104-158, :207-343) with the library's stages
    (or, for checking, with the float64 oracle's)."""
    pre, scan, post = stages or _cuda_stages()
    B, T, _ = x.shape
    xn = rmsnorm(x, w["norm_scale"])
    qp = xn @ w["wq"]
    if kv_share:  # one wide projection: the first Dk channels of every head are the key
        vp = xn @ w["w_kv"]
        kp = vp.view(B, T, H, Dv)[..., :Dk].reshape(B, T, H * Dk)
    else:
        kp, vp = xn @ w["wk"], xn @ w["wv"]
    q, k, v, beta, gate = pre(qp, kp, vp, w["q_conv"], w["k_conv"], w["v_conv"], xn @ w["w_a"], xn @ w["w_beta"],
                              w["A_log"], w["dt_bias"], H, Dk, Dv)
    return x + post(scan(q, k, v, beta, gate, chunk), xn @ w["w_out_gate"], w["o_norm_scale"]) @ w["wo"]


@pytest.mark.parametrize("fixture", ["gdn_fla_grad_kvshare.npz", "gdn_fla_grad_nokvshare.npz"])
@pytest.mark.parametrize("chunk", [64, 0])
def test_gated_deltanet_block_matches_reference_fixture(fixture, chunk):
    z = np.load(os.path.join(G, fixture))
    H, Dk, Dv = int(z["heads"][0]), int(z["d_k"][0]), int(z["d_v"][0])
    kv_share = bool(z["kv_share"][0])
    names = ["norm_scale", "wq", "q_conv", "k_conv", "v_conv", "w_a", "A_log", "dt_bias", "w_beta", "w_out_gate",
             "o_norm_scale", "wo", "final_norm_scale"] + (["w_kv"] if kv_share else ["wk", "wv"])
    w = {n: torch.from_numpy(z[n]).to(DEV).contiguous().requires_grad_(True) for n in names}
    x = torch.from_numpy(z["input"]).to(DEV)[None]
    y = rmsnorm(gdn_block_forward(x, w, H, Dk, Dv, kv_share, chunk), w["final_norm_scale"])
    loss = y.pow(2).mean()
    loss.backward()
    torch.cuda.synchronize()
    # the reference test's own bound: max-abs 1e-3 on the hidden state and on every gradient
    err = (y.detach().cpu() - torch.from_numpy(z["expected_x_hidden"])).abs().max().item()
    assert err <= 1e-3, ("hidden", err)
    assert abs(loss.item() - float(z["loss"][0])) <= 1e-4
    worst = {}
    for n in names:
        want = torch.from_numpy(z[n + "_grad"])
        got = w[n].grad.detach().cpu()
        assert got.shape == want.shape, (n, got.shape, want.shape)
        worst[n] = ((got - want).abs().max().item(), want.abs().max().item())
    bad = {n: e for n, e in worst.items() if e[0] > 1e-3 or e[0] > 2e-3 * max(e[1], 1e-6) + 1e-6}
    assert not bad, bad


@pytest.mark.parametrize("fixture", ["gdn_fla_grad_kvshare.npz", "gdn_fla_grad_nokvshare.npz"])
def test_gated_deltanet_block_gradients_against_oracle(fixture):
    """The fixture's loss sits behind a final RMSNorm, which makes its weight gradients tiny (1e-7) and the reference's
    1e-3 bound loose.  Same block and weights, but a random cotangent on the block output and no final norm: every
    weight gradient within 1e-3 (relative to its largest entry) of the float64 oracle composition."""
    z = np.load(os.path.join(G, fixture))
    H, Dk, Dv = int(z["heads"][0]), int(z["d_k"][0]), int(z["d_v"][0])
    kv_share = bool(z["kv_share"][0])
    names = ["norm_scale", "wq", "q_conv", "k_conv", "v_conv", "w_a", "A_log", "dt_bias", "w_beta", "w_out_gate",
             "o_norm_scale", "wo"] + (["w_kv"] if kv_share else ["wk", "wv"])
    x = torch.from_numpy(z["input"])[None]
    cot = torch.randn(x.shape, generator=torch.Generator().manual_seed(3), dtype=torch.float64)
    w64 = {n: torch.from_numpy(z[n]).double().requires_grad_(True) for n in names}
    (gdn_block_forward(x.double(), w64, H, Dk, Dv, kv_share, 64, _oracle_stages()) * cot).sum().backward()
    w = {n: torch.from_numpy(z[n]).to(DEV).contiguous().requires_grad_(True) for n in names}
    out = gdn_block_forward(x.to(DEV), w, H, Dk, Dv, kv_share, 64)
    (out * cot.float().to(DEV)).sum().backward()
    torch.cuda.synchronize()
    bad = {}
    for n in names:
        want, got = w64[n].grad, w[n].grad.detach().double().cpu()
        e = (got - want).abs().max().item()
        if e > 1e-3 * want.abs().max().item():
            bad[n] = (e, want.abs().max().item())
    assert not bad, bad


def test_gated_deltanet_bidirectional_composition():
    """bidirectional = the same block on the sequence and on its time reversal, outputs added
    (arch/blocks_gated_deltanet.go:109-147, all positions valid): a composition on the caller's side, checked here
    against the same composition of the float64 oracle stages."""
    z = np.load(os.path.join(G, "gdn_fla_grad_nokvshare.npz"))
    H, Dk, Dv = int(z["heads"][0]), int(z["d_k"][0]), int(z["d_v"][0])
    names = ["norm_scale", "wq", "wk", "wv", "q_conv", "k_conv", "v_conv", "w_a", "A_log", "dt_bias", "w_beta", "w_out_gate",
             "o_norm_scale", "wo"]
    x = torch.from_numpy(z["input"])[None]

    def both_ways(xx, ww, stages):  # delta(x) + reverse(delta(reverse(x))), residual added once
        delta = lambda t: gdn_block_forward(t, ww, H, Dk, Dv, False, 64, stages) - t
        return xx + delta(xx) + delta(xx.flip(1).contiguous()).flip(1)

    with torch.no_grad():
        got = both_ways(x.to(DEV), {n: torch.from_numpy(z[n]).to(DEV).contiguous() for n in names}, None)
        want = both_ways(x.double(), {n: torch.from_numpy(z[n]).double() for n in names}, _oracle_stages())
    assert (got.double().cpu() - want).abs().max().item() <= 1e-4 * max(1.0, want.abs().max().item())


# ---------------------------------------------------------------- Mamba-3 canonical block
class M3Conv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return ops.mamba3_block_conv(x, w)

    @staticmethod
    def backward(ctx, dy):
        g = ops.mamba3_block_conv_backward(*ctx.saved_tensors, dy.contiguous())
        return g["dx"], g["dw"]


class M3BC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, bp, cp, bs, cs, bb, cb, G_, N):
        ctx.save_for_backward(bp, cp, bs, cs)
        ctx.dims = (G_, N)
        return ops.mamba3_block_bc(bp, cp, bs, cs, bb, cb, G_, N)

    @staticmethod
    def backward(ctx, db, dc):
        G_, N = ctx.dims
        g = ops.mamba3_block_bc_backward(*ctx.saved_tensors, db.contiguous(), dc.contiguous(), G_, N)
        return g["db_proj"], g["dc_proj"], g["db_scale"], g["dc_scale"], g["db_bias"], g["dc_bias"], None, None


class M3Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dt, lam, theta, a_log, b, c):
        ctx.save_for_backward(x, dt, lam, theta, a_log, b, c)
        return ops.mamba3_selective_scan(x, dt, lam, theta, a_log, b, c)

    @staticmethod
    def backward(ctx, dy):
        g = ops.mamba3_selective_scan_backward(*ctx.saved_tensors, dy.contiguous())
        return g["dx"], g["ddt"], g["dlambda"], g["dtheta"], g["da_log"], g["db"], g["dc"]


class M3Post(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, z, pn):
        ctx.save_for_backward(y, z, pn)
        return ops.mamba3_block_post(y, z, pn)

    @staticmethod
    def backward(ctx, dout):
        g = ops.mamba3_block_post_backward(*ctx.saved_tensors, dout.contiguous())
        return g["dy"], g["dz"], g["dpost_norm"]


def test_mamba3_canonical_block_matches_reference_module():
    """mamba3_canonical_block_impl (gpu/ir.cpp:2034-2105): pre-norm, x projection, causal depthwise conv, low-rank
    dt / lambda / theta, B/C norm + bias, scan, post-norm x gate, output projection, residual."""
    z = np.load(os.path.join(G, "mamba3_full_block_torch.npz"))
    B, T, Dm, D, N, Gr, rank, K = (int(v) for v in z["dims"])
    pnames = [k[2:] for k in z.files if k.startswith("w:")]
    w = {n: torch.from_numpy(z["w:" + n]).float().to(DEV).contiguous().requires_grad_(True) for n in pnames}
    x = torch.from_numpy(z["input"]).float().to(DEV)
    xn = rmsnorm(x, w["pre_norm.weight"])
    xb = M3Conv.apply((xn @ w["w_x.weight"]).contiguous(), w["conv_weight"])
    dt = (xb @ w["w_dt_low.weight"]) @ w["w_dt_high.weight"] + w["dt_bias"]
    lam = (xb @ w["w_lambda_low.weight"]) @ w["w_lambda_high.weight"]
    theta = ((xb @ w["w_theta_low.weight"]) @ w["w_theta_high.weight"]).view(B, T, D, N // 2)
    b, c = M3BC.apply((xb @ w["w_B.weight"]).contiguous(), (xb @ w["w_C.weight"]).contiguous(), w["B_norm.weight"],
                      w["C_norm.weight"], w["B_bias"], w["C_bias"], Gr, N)
    y = M3Scan.apply(xb, dt.contiguous(), lam.contiguous(), theta.contiguous(), w["A_log"], b, c)
    out = x + M3Post.apply(y, (xn @ w["w_gate.weight"]).contiguous(), w["post_norm.weight"]) @ w["w_out.weight"]
    loss = out.pow(2).mean()
    loss.backward()
    torch.cuda.synchronize()
    want = torch.from_numpy(z["output"])
    assert (out.detach().double().cpu() - want).abs().max().item() <= 1e-4 * max(1.0, want.abs().max().item())
    bad = {}
    for n in pnames:
        gw = torch.from_numpy(z["g:" + n])
        got = w[n].grad.detach().double().cpu()
        e = (got - gw).abs().max().item()
        if e > 1e-3 * max(gw.abs().max().item(), 1e-6) + 1e-7:
            bad[n] = (e, gw.abs().max().item())
    assert not bad, bad
