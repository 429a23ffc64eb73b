"""Mamba-3 exponential-trapezoidal selective scan: CPU restatement (torch, CPU).

TEST INFRASTRUCTURE ONLY - see ``oracle/__init__.py``.

Layouts follow the reference operator ``OP_MAMBA3_SELECTIVE_SCAN``
(``arch/ir.go:528-553``):

    x, dt_raw, lambda_raw : [B, T, D]     theta : [B, T, D, N/2]
    a_log : [D, N]                         b_proj, c_proj : [B, T, G, N]
    y : [B, T, D]

Recurrence (gpu/cuda_kernels/mamba3_selective_scan_fwd_v2_emit.cu:65-115,
train/gpu_trainer_mamba3_test.go:612-690):

    dt = softplus(dt_raw); lam = sigmoid(lambda_raw); A = -exp(a_log)
    phi_t = phi_{t-1} + dt_t * theta_t
    Brot = R^T(phi) B ; Crot = R^T(phi) C     (even' = c e + s o ; odd' = -s e + c o)
    alpha = exp(dt A); beta = (1 - lam) dt alpha; gamma = lam dt
    h_t = alpha h_{t-1} + gamma Brot_t x_t + [t>0] beta Brot_{t-1} x_{t-1}
    y_t = sum_n h_t[n] Crot_t[n]
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def rotate_pairs(values: torch.Tensor, phi: torch.Tensor) -> torch.Tensor:
    """R^T(phi) on consecutive (even, odd) pairs - mamba3_selective_scan_common.cuh:39-48."""
    pairs = values.reshape(*values.shape[:-1], -1, 2)
    e, o = pairs[..., 0], pairs[..., 1]
    c, s = torch.cos(phi), torch.sin(phi)
    return torch.stack((c * e + s * o, -s * e + c * o), dim=-1).flatten(-2)


def _expand_groups(p: torch.Tensor, D: int) -> torch.Tensor:
    """[B,T,G,N] -> [B,T,D,N] with g = d // (D/G)."""
    G = p.shape[2]
    return p.repeat_interleave(D // G, dim=2)


def scan_forward(x, dt_raw, lambda_raw, theta, a_log, b_proj, c_proj, return_state=False):
    """Sequential recurrence; autograd-friendly.  Returns y [B,T,D] (and h_T [B,D,N])."""
    B, T, D = x.shape
    N = a_log.shape[-1]
    dt = F.softplus(dt_raw)
    lam = torch.sigmoid(lambda_raw)
    A = -torch.exp(a_log)
    phi = torch.cumsum(dt[..., None] * theta, dim=1)
    b_rot = rotate_pairs(_expand_groups(b_proj, D), phi)
    c_rot = rotate_pairs(_expand_groups(c_proj, D), phi)
    h = x.new_zeros((B, D, N))
    ys = []
    for t in range(T):
        alpha = torch.exp(dt[:, t, :, None] * A)
        cur = (lam[:, t] * dt[:, t] * x[:, t])[..., None] * b_rot[:, t]
        h = alpha * h + cur
        if t > 0:
            beta = ((1.0 - lam[:, t]) * dt[:, t])[..., None] * alpha
            h = h + beta * b_rot[:, t - 1] * x[:, t - 1, :, None]
        ys.append((h * c_rot[:, t]).sum(-1))
    y = torch.stack(ys, dim=1) if ys else x.new_zeros((B, 0, D))
    return (y, h) if return_state else y


def scan_vjp(x, dt_raw, lambda_raw, theta, a_log, b_proj, c_proj, dy):
    """Closed-form VJP - restates mamba3MIMOCPUForwardBackward
    (train/gpu_trainer_mamba3_test.go:612-808) / the MLX closed form
    (gpu/ir.cpp:1526-1623) with an arbitrary cotangent ``dy`` [B,T,D].

    Returns (y, dict(dx, ddt, dlambda, dtheta, da_log, db, dc)).
    """
    B, T, D = x.shape
    N = a_log.shape[-1]
    G = b_proj.shape[2]
    K = N // 2
    dt = F.softplus(dt_raw)
    lam = torch.sigmoid(lambda_raw)
    A = -torch.exp(a_log)  # [D,N]
    phi = torch.cumsum(dt[..., None] * theta, dim=1)  # [B,T,D,K]
    b_rot = rotate_pairs(_expand_groups(b_proj, D), phi)
    c_rot = rotate_pairs(_expand_groups(c_proj, D), phi)
    alpha = torch.exp(dt[..., None] * A)  # [B,T,D,N]

    # forward, keeping h before/after every step
    h = x.new_zeros((B, D, N))
    h_before = x.new_zeros((B, T, D, N))
    h_after = x.new_zeros((B, T, D, N))
    for t in range(T):
        h_before[:, t] = h
        cur = (lam[:, t] * dt[:, t] * x[:, t])[..., None] * b_rot[:, t]
        h = alpha[:, t] * h + cur
        if t > 0:
            h = h + ((1.0 - lam[:, t]) * dt[:, t])[..., None] * alpha[:, t] * b_rot[:, t - 1] * x[:, t - 1, :, None]
        h_after[:, t] = h
    y = (h_after * c_rot).sum(-1)

    dx = torch.zeros_like(x)
    ddelta = torch.zeros_like(x)
    dlam = torch.zeros_like(x)
    da_log = torch.zeros_like(a_log)
    g_brot = torch.zeros_like(b_rot)
    g_crot = dy[..., None] * h_after
    dh_next = x.new_zeros((B, D, N))
    for t in range(T - 1, -1, -1):
        up = dh_next + dy[:, t, :, None] * c_rot[:, t]  # [B,D,N]
        lt, dtt, xt = lam[:, t, :, None], dt[:, t, :, None], x[:, t, :, None]
        a, bv = alpha[:, t], b_rot[:, t]
        dx[:, t] += (lt * dtt * bv * up).sum(-1)
        g_brot[:, t] += lt * dtt * xt * up
        delta_term = A * a * h_before[:, t]
        alog_term = dtt * a * A * h_before[:, t]
        if t > 0:
            px = x[:, t - 1, :, None]
            pb = b_rot[:, t - 1]
            pin = pb * px
            bni = (1.0 - lt) * dtt * a
            dx[:, t - 1] += (bni * pb * up).sum(-1)
            g_brot[:, t - 1] += bni * px * up
            dlam[:, t] = ((-dtt * a * pin + dtt * bv * xt) * up).sum(-1)
            delta_term = delta_term + (1.0 - lt) * (a + dtt * A * a) * pin
            alog_term = alog_term + (1.0 - lt) * dtt * dtt * a * A * pin
        else:
            dlam[:, t] = (dtt * bv * xt * up).sum(-1)
        ddelta[:, t] += ((delta_term + lt * bv * xt) * up).sum(-1)
        da_log += (alog_term * up).sum(0)
        dh_next = a * up
    dlam = dlam * lam * (1.0 - lam)

    # rotation VJP (train/gpu_trainer_mamba3_test.go:752-786)
    c, s = torch.cos(phi), torch.sin(phi)

    def unrot(gr):
        p = gr.reshape(B, T, D, K, 2)
        g0, g1 = p[..., 0], p[..., 1]
        return torch.stack((c * g0 - s * g1, s * g0 + c * g1), dim=-1).flatten(-2)

    def group_sum(gfull):
        return gfull.reshape(B, T, G, D // G, N).sum(3)

    db = group_sum(unrot(g_brot))
    dc = group_sum(unrot(g_crot))
    br, cr = b_rot.reshape(B, T, D, K, 2), c_rot.reshape(B, T, D, K, 2)
    gb, gc = g_brot.reshape(B, T, D, K, 2), g_crot.reshape(B, T, D, K, 2)
    g_phi = br[..., 1] * gb[..., 0] - br[..., 0] * gb[..., 1] + cr[..., 1] * gc[..., 0] - cr[..., 0] * gc[..., 1]
    carry = torch.flip(torch.cumsum(torch.flip(g_phi, [1]), 1), [1])  # suffix sum over t
    dtheta = carry * dt[..., None]
    ddelta = ddelta + (carry * theta).sum(-1)
    ddt = ddelta * torch.sigmoid(dt_raw)
    return y, dict(dx=dx, ddt=ddt, dlambda=dlam, dtheta=dtheta, da_log=da_log, db=db, dc=dc)


def scan_grads_autograd(x, dt_raw, lambda_raw, theta, a_log, b_proj, c_proj, dy):
    """Same gradients through torch autograd on ``scan_forward`` (cross-check of ``scan_vjp``)."""
    leaves = [t.detach().clone().requires_grad_(True)
              for t in (x, dt_raw, lambda_raw, theta, a_log, b_proj, c_proj)]
    y = scan_forward(*leaves)
    g = torch.autograd.grad((y * dy).sum(), leaves)
    names = ("dx", "ddt", "dlambda", "dtheta", "da_log", "db", "dc")
    return y.detach(), dict(zip(names, g))
