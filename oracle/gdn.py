"""Gated delta rule: CPU restatement of the reference algorithms (torch, CPU).

TEST INFRASTRUCTURE ONLY - see ``oracle/__init__.py``.

Layouts follow the reference operator ``OP_GATED_DELTA_SCAN``
(``arch/ir.go:586-603``, ``gpu/ir.cpp:4633-4654``):

    q, k : [B, T, H, Dk]     v : [B, T, H, Dv]     beta, gate : [B, T, H]
    out  : [B, T, H, Dv]     state : [B, H, Dk, Dv]

``gate`` is the multiplicative decay in (0, 1].  The reference operator has no
initial-state input and does not return the final state; both are exposed here
(``h0`` / second return value) because the recurrence defines them.

All functions compute in the dtype of ``q`` (use float64 tensors for the
checker, float32 tensors for the timed CPU baseline).
"""

from __future__ import annotations

import torch

# gpu/ir.cpp:35-37
GATE_FLOOR = 1e-30
EXP_CLAMP_MIN = -80.0
EXP_CLAMP_MAX = 0.0


def stable_exp_nonpos(x: torch.Tensor) -> torch.Tensor:
    """exp(clamp(x, -80, 0)) - gpu/ir.cpp:893-905."""
    return torch.exp(torch.clamp(x, EXP_CLAMP_MIN, EXP_CLAMP_MAX))


def decode_step(state, q, k, v, beta, gate):
    """One token of the recurrence on a persistent state.

    Loop body of ``gated_delta_scan_naive`` (gpu/ir.cpp:2334-2345):
    decay, predict, delta update, read-out.

    state [N,H,Dk,Dv]; q,k [N,H,Dk]; v [N,H,Dv]; beta,gate [N,H].
    Returns (out [N,H,Dv], new_state).
    """
    state = gate[..., None, None] * state
    pred = torch.einsum("nhk,nhkv->nhv", k, state)
    err_scaled = (v - pred) * beta[..., None]
    state = state + k[..., :, None] * err_scaled[..., None, :]
    out = torch.einsum("nhk,nhkv->nhv", q, state)
    return out, state


def scan_naive(q, k, v, beta, gate, h0=None):
    """Token-by-token recurrence - gpu/ir.cpp:2314-2350.

    Returns (out [B,T,H,Dv], final_state [B,H,Dk,Dv]).
    """
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    state = q.new_zeros((B, H, Dk, Dv)) if h0 is None else h0
    outs = []
    for t in range(T):
        o, state = decode_step(state, q[:, t], k[:, t], v[:, t], beta[:, t], gate[:, t])
        outs.append(o)
    if outs:
        out = torch.stack(outs, dim=1)
    else:
        out = q.new_zeros((B, 0, H, Dv))
    return out, state


def solve_strictly_lower(raw: torch.Tensor) -> torch.Tensor:
    """X = (I - raw)^-1 for strictly-lower ``raw`` [..., C, C].

    Column-parallel forward substitution of
    gpu/cuda_kernels/gated_delta_chunk_solve.cu:16-26 (row i of X is
    e_i + sum_{j<i} raw[i,j] * X[j,:]); identical to the row-wise CPU fallback
    of gpu/ir.cpp:2464-2479.
    """
    C = raw.shape[-1]
    rows = []
    for i in range(C):
        e = torch.zeros(raw.shape[:-2] + (C,), dtype=raw.dtype)
        e[..., i] = 1.0
        if i > 0:
            prev = torch.stack(rows, dim=-2)  # [..., i, C]
            e = e + torch.einsum("...j,...jc->...c", raw[..., i, :i], prev)
        rows.append(e)
    return torch.stack(rows, dim=-2)


def solve_strictly_lower_vjp(solved: torch.Tensor, cot: torch.Tensor) -> torch.Tensor:
    """tril(T^T . cot . T^T, -1) - gpu/gated_delta_cuda_primitive.cpp:104-132."""
    tt = solved.transpose(-1, -2)
    return torch.tril(tt @ cot @ tt, diagonal=-1)


def scan_chunked(q_in, k_in, v_in, beta_in, gate_in, chunk_size=64, h0=None, solve="substitution"):
    """Chunked WY/UT form, op for op after gpu/ir.cpp:2352-2550.

    ``h0`` (not in the reference, which starts from zero at :2502) seeds the
    state.  ``solve`` = "substitution" follows the CUDA primitive's forward
    substitution; "triangular" uses a library triangular solve (same matrix;
    faster for the timed CPU baseline).
    Returns (out [B,T,H,Dv], final_state [B,H,Dk,Dv]).
    """
    if chunk_size <= 1:
        return scan_naive(q_in, k_in, v_in, beta_in, gate_in, h0)
    B, T, H, Dk = q_in.shape
    Dv = v_in.shape[-1]
    dt = q_in.dtype
    C = chunk_size
    pad = (C - (T % C)) % C
    Tp = T + pad
    n = Tp // C

    q = q_in.transpose(1, 2)
    k = k_in.transpose(1, 2)
    v = v_in.transpose(1, 2)
    beta = beta_in.transpose(1, 2)
    gate = gate_in.transpose(1, 2)
    if pad:
        q = torch.cat([q, q.new_zeros((B, H, pad, Dk))], 2)
        k = torch.cat([k, k.new_zeros((B, H, pad, Dk))], 2)
        v = torch.cat([v, v.new_zeros((B, H, pad, Dv))], 2)
        beta = torch.cat([beta, beta.new_zeros((B, H, pad))], 2)
        gate = torch.cat([gate, gate.new_ones((B, H, pad))], 2)
    gate = torch.clamp(gate, min=GATE_FLOOR)

    q = q.reshape(B, H, n, C, Dk)
    k = k.reshape(B, H, n, C, Dk)
    v = v.reshape(B, H, n, C, Dv)
    beta = beta.reshape(B, H, n, C)
    gate = gate.reshape(B, H, n, C)

    v_beta = v * beta[..., None]
    k_beta = k * beta[..., None]
    log_decay = torch.cumsum(torch.log(gate), 3)
    decay_exp = stable_exp_nonpos(log_decay)

    idx = torch.arange(C)
    strict = (idx[:, None] > idx[None, :]).to(dt)
    lower = (idx[:, None] >= idx[None, :]).to(dt)
    decay_delta = stable_exp_nonpos(log_decay[..., :, None] - log_decay[..., None, :])

    raw_attn = -(k_beta @ k.transpose(-1, -2)) * decay_delta * strict
    if solve == "substitution":
        solve_attn = solve_strictly_lower(raw_attn)
    else:
        eye = torch.eye(C, dtype=dt)
        solve_attn = torch.linalg.solve_triangular(eye - raw_attn, eye.expand_as(raw_attn), upper=False)

    k_cumsum = solve_attn @ v_beta
    k_cumdecay = solve_attn @ (k_beta * decay_exp[..., None])
    causal_attn = (q @ k.transpose(-1, -2)) * decay_delta * lower

    state = q.new_zeros((B, H, Dk, Dv)) if h0 is None else h0
    outs = []
    for c in range(n):
        q_i, k_i = q[:, :, c], k[:, :, c]
        v_i, kd_i = k_cumsum[:, :, c], k_cumdecay[:, :, c]
        ld = log_decay[:, :, c]
        v_new = v_i - kd_i @ state
        o_inter = (q_i * stable_exp_nonpos(ld)[..., None]) @ state
        outs.append(o_inter + causal_attn[:, :, c] @ v_new)
        last = ld[..., -1]
        carry = stable_exp_nonpos(last[..., None] - ld)
        upd = (k_i * carry[..., None]).transpose(-1, -2) @ v_new
        state = state * stable_exp_nonpos(last)[..., None, None] + upd
    out = torch.stack(outs, 2).reshape(B, H, Tp, Dv)[:, :, :T]
    return out.transpose(1, 2).contiguous(), state


def scan_grads(q, k, v, beta, gate_or_g, d_out, d_final_state=None, h0=None,
               gate_is_log=False, chunk_size=0):
    """Forward + all gradients by autograd through the restated recurrence.

    The reference has no hand-written backward for this op: MLX autograd
    differentiates ``gated_delta_scan_*`` op by op (only the triangular solve
    has a custom VJP, gpu/gated_delta_cuda_primitive.cpp:104-132).  This does
    the same with torch autograd.  ``gate_is_log``: the 5th input is the log
    decay g (gate = exp(g)) and the returned gradient is with respect to g.
    Returns dict(out, state, dq, dk, dv, dbeta, dgate, dh0).
    """
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v, beta, gate_or_g)]
    h0l = None if h0 is None else h0.detach().clone().requires_grad_(True)
    gate = torch.exp(leaves[4]) if gate_is_log else leaves[4]
    if chunk_size and chunk_size > 1:
        out, state = scan_chunked(leaves[0], leaves[1], leaves[2], leaves[3], gate, chunk_size, h0l)
    else:
        out, state = scan_naive(leaves[0], leaves[1], leaves[2], leaves[3], gate, h0l)
    loss = (out * d_out).sum()
    if d_final_state is not None:
        loss = loss + (state * d_final_state).sum()
    wrt = leaves + ([h0l] if h0l is not None else [])
    grads = torch.autograd.grad(loss, wrt, allow_unused=True)
    res = dict(out=out.detach(), state=state.detach(), dq=grads[0], dk=grads[1], dv=grads[2],
               dbeta=grads[3], dgate=grads[4], dh0=grads[5] if h0l is not None else None)
    return res
