"""CPU restatement of the element-wise stages of mixlab's canonical Mamba-3 block around the
scan - TEST INFRASTRUCTURE ONLY (imported by tests/, smoke() and bench.py's CPU legs).

Follows mamba3_canonical_block_impl, gpu/ir.cpp:2034-2105 of the reference:

  conv   x_branch = causal_depthwise_conv1d(x_proj, conv_w)          (gpu/ir.cpp:1397-1425: weight [D, K],
         tap k multiplies x[t-k], zero history, no activation)
  bc     b = RMSNorm(b_proj rows of N, b_norm_scale, eps) + b_bias,  same for c           (:2089-2094)
  post   out = RMSNorm(y rows of D, post_norm, eps) * z * sigmoid(z)                      (:2099-2102)

The projections (matrix products) on either side stay with the caller.  Pinned by
tests/golden/mamba3_block_stages.json (the reference's own scalar helpers).  Gradients come from
torch autograd over these functions in float64.
"""
from __future__ import annotations

import torch


def depthwise_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [B,T,D], w [D,K] -> sum_k w[:,k] * x[t-k]."""
    B, T, D = x.shape
    out = torch.zeros_like(x)
    for k in range(min(w.shape[1], T)):
        out[:, k:] = out[:, k:] + x[:, :T - k] * w[:, k]
    return out


def rms_norm(x: torch.Tensor, scale: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * scale


def bc_norm(b_proj, c_proj, b_scale, c_scale, b_bias, c_bias, G, N, eps=1e-5):
    """b_proj, c_proj [B,T,G*N] -> b, c [B,T,G,N]."""
    B, T, _ = b_proj.shape
    b = rms_norm(b_proj.reshape(B, T, G, N), b_scale, eps) + b_bias.reshape(G, N)
    c = rms_norm(c_proj.reshape(B, T, G, N), c_scale, eps) + c_bias.reshape(G, N)
    return b, c


def post(y, z, post_norm, eps=1e-5):
    """y, z [B,T,D] -> RMSNorm(y, post_norm, eps) * z * sigmoid(z)."""
    return rms_norm(y, post_norm, eps) * z * torch.sigmoid(z)
