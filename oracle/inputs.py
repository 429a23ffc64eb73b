"""Seeded synthetic inputs for the benchmark configurations.

TEST INFRASTRUCTURE ONLY - see ``oracle/__init__.py``.

All draws come from a CPU ``torch.Generator`` so that the CPU checker and the
GPU path see identical bits.  Draw order within a config is fixed and listed
in each function.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


def gdn_inputs(B, T, H, Dk, Dv, seed=0, io_dtype=torch.float32, with_grad_out=False, with_h0=False):
    """q,k,v ~ N(0,1) (q,k L2-normalised per head vector), beta = sigmoid(N(0,1)),
    g = -softplus(N(0,1)) (log decay).  Draw order: q, k, v, beta, g, [dO], [h0], [dhT].

    q,k,v,(dO) are rounded to ``io_dtype``; beta, g and states stay fp32.
    Returns a dict of fp32/io_dtype CPU tensors.
    """
    g = _gen(seed)
    q = torch.randn(B, T, H, Dk, generator=g)
    k = torch.randn(B, T, H, Dk, generator=g)
    v = torch.randn(B, T, H, Dv, generator=g)
    q = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    k = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g))
    glog = -F.softplus(torch.randn(B, T, H, generator=g))
    out = dict(q=q.to(io_dtype), k=k.to(io_dtype), v=v.to(io_dtype), beta=beta, g=glog)
    if with_grad_out:
        out["d_out"] = torch.randn(B, T, H, Dv, generator=g).to(io_dtype)
    if with_h0:
        out["h0"] = 0.1 * torch.randn(B, H, Dk, Dv, generator=g)
        out["d_state"] = 0.1 * torch.randn(B, H, Dk, Dv, generator=g)
    return out


def gdn_decode_inputs(N, H, Dk, Dv, steps, seed=2, io_dtype=torch.bfloat16):
    """state ~ N(0, 0.02) fp32 [N,H,Dk,Dv]; per step q,k,v (q,k normalised),
    beta = sigmoid(N(0,1)), g = -softplus(N(0,1)).  Draw order: state, then
    q, k, v, beta, g each with a leading [steps] axis."""
    g = _gen(seed)
    state = 0.02 * torch.randn(N, H, Dk, Dv, generator=g)
    q = torch.randn(steps, N, H, Dk, generator=g)
    k = torch.randn(steps, N, H, Dk, generator=g)
    v = torch.randn(steps, N, H, Dv, generator=g)
    q = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    k = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    beta = torch.sigmoid(torch.randn(steps, N, H, generator=g))
    glog = -F.softplus(torch.randn(steps, N, H, generator=g))
    return dict(state=state, q=q.to(io_dtype), k=k.to(io_dtype), v=v.to(io_dtype), beta=beta, g=glog)


def mamba3_inputs(B, T, nheads, headdim, N, G=1, seed=3, io_dtype=torch.float32, per_head=True):
    """x [B,T,D], B/C [B,T,G,N] ~ N(0,1); dt_raw ~ N(-2, 0.5) (kernel applies
    softplus); a_log ~ U(log 1, log 16); theta ~ U(-pi, pi); lambda_raw ~ N(0,1);
    dY ~ N(0,1).  Draw order: x, b, c, dt_raw, a_log, theta, lambda_raw, dy.

    ``per_head`` True: dt_raw, lambda_raw [B,T,nheads], theta [B,T,nheads]
    (one angle rate shared by all state pairs of the head), a_log [nheads].
    False: the reference's per-channel layout dt_raw, lambda_raw [B,T,D],
    theta [B,T,D,N/2], a_log [D,N].
    """
    g = _gen(seed)
    D = nheads * headdim
    x = torch.randn(B, T, D, generator=g).to(io_dtype)
    b = torch.randn(B, T, G, N, generator=g).to(io_dtype)
    c = torch.randn(B, T, G, N, generator=g).to(io_dtype)
    if per_head:
        dt_raw = -2.0 + 0.5 * torch.randn(B, T, nheads, generator=g)
        a_log = math.log(1.0) + (math.log(16.0) - math.log(1.0)) * torch.rand(nheads, generator=g)
        theta = (2.0 * torch.rand(B, T, nheads, generator=g) - 1.0) * math.pi
        lam = torch.randn(B, T, nheads, generator=g)
    else:
        dt_raw = -2.0 + 0.5 * torch.randn(B, T, D, generator=g)
        a_log = math.log(16.0) * torch.rand(D, N, generator=g)
        theta = (2.0 * torch.rand(B, T, D, N // 2, generator=g) - 1.0) * math.pi
        lam = torch.randn(B, T, D, generator=g)
    dy = torch.randn(B, T, D, generator=g).to(io_dtype)
    return dict(x=x, b=b, c=c, dt_raw=dt_raw, a_log=a_log, theta=theta, lambda_raw=lam, dy=dy,
                nheads=nheads, headdim=headdim)


def mamba3_expand_per_head(inp):
    """Broadcast a per-head input dict to the reference's per-channel layout."""
    H, P = inp["nheads"], inp["headdim"]
    N = inp["b"].shape[-1]
    out = dict(inp)
    out["dt_raw"] = inp["dt_raw"].repeat_interleave(P, dim=-1)
    out["lambda_raw"] = inp["lambda_raw"].repeat_interleave(P, dim=-1)
    out["theta"] = inp["theta"].repeat_interleave(P, dim=-1)[..., None].expand(-1, -1, -1, N // 2).contiguous()
    out["a_log"] = inp["a_log"].repeat_interleave(P)[:, None].expand(-1, N).contiguous()
    return out
