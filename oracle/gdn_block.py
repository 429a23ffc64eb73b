"""CPU restatement of the element-wise stages of mixlab's gated_deltanet block around the
scan - TEST INFRASTRUCTURE ONLY (imported by tests/, smoke() and bench.py's CPU legs).

Follows emitGatedDeltaNetDeltaIR, arch/blocks_gated_deltanet.go:207-343 of the reference:

  pre   q_seq = SiLU(conv4(q_proj)), k_seq = SiLU(conv4(k_proj)), v = SiLU(conv4(v_proj))
        (emitGatedDeltaNetShortConv1D, :345-368: causal, 4 taps, tap j multiplies x[t-j], weight [4, C])
        q = RMSNorm(q_seq, ones, 1e-6) / dk,  k = RMSNorm(k_seq, ones, 1e-6) / sqrt(dk)      (:308-316)
        gate = exp(-softplus(a_raw + dt_bias) * exp(A_log)),  beta = sigmoid(b_raw)          (:318-330)
  post  y = RMSNorm(o, o_norm, 1e-5) * SiLU(z)                                               (:333-341)

The projections on either side are plain matrix products and stay with the caller.
Pinned by tests/golden/gdn_block_stages.json (the reference's own scalar helpers).
Gradients come from torch autograd over these functions in float64.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def short_conv_silu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [B,T,C], w [4,C] -> SiLU(sum_j w[j] * x[t-j])  (zero history)."""
    B, T, C = x.shape
    acc = torch.zeros_like(x)
    for tap in range(4):
        if tap < T:
            acc[:, tap:] = acc[:, tap:] + x[:, :T - tap] * w[tap]
    return F.silu(acc)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)


def block_pre(q_proj, k_proj, v_proj, conv_q, conv_k, conv_v, a_raw, b_raw, a_log, dt_bias, H, Dk, Dv, gate_is_log=False):
    """Returns q [B,T,H,Dk], k [B,T,H,Dk], v [B,T,H,Dv], beta [B,T,H], gate [B,T,H] (or its log)."""
    B, T, _ = q_proj.shape
    q = rms_unit(short_conv_silu(q_proj, conv_q).reshape(B, T, H, Dk), 1e-6) / Dk
    k = rms_unit(short_conv_silu(k_proj, conv_k).reshape(B, T, H, Dk), 1e-6) / math.sqrt(Dk)
    v = short_conv_silu(v_proj, conv_v).reshape(B, T, H, Dv)
    log_gate = -F.softplus(a_raw + dt_bias) * torch.exp(a_log)
    beta = torch.sigmoid(b_raw)
    return q, k, v, beta, (log_gate if gate_is_log else torch.exp(log_gate))


def block_post(o, z, o_norm):
    """o [B,T,H,Dv], z [B,T,H*Dv] (pre-activation of the output gate), o_norm [Dv] -> y [B,T,H*Dv]."""
    B, T, H, Dv = o.shape
    y = rms_unit(o, 1e-5) * o_norm * F.silu(z.reshape(B, T, H, Dv))
    return y.reshape(B, T, H * Dv)
