"""Size-independent properties of the CUDA paths at the full benchmark sizes (where the CPU oracle would take
minutes): splitting a sequence in two with the state handed over, independence of the (batch, head) problems,
backward from saved intermediates against the recomputing backward, tensor-copy staging against per-thread staging.
Every property compares two runs of the same kernels on the same data, so the bar is bit-exact equality
(fp32 hand-over of the state and fixed-order reductions make the two sides the same arithmetic).  One sequence of the
benchmark configuration is also checked against the float64 oracle itself (about 12 s of CPU time).

Sizes: gated delta rule B=8, T=4096, H=16, d_k=d_v=128, chunk 64, bf16 I/O; recurrent decode 256 sequences x 16
heads; Mamba-3 B=8, T=4096, 32 heads x 64, d_state 128, bf16 I/O."""
import math

import pytest
import torch

from mixlab_b200 import _lib, ops
from oracle import gdn, inputs
from tests.util import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _gdn_full(B=8, T=4096, H=16, D=128, seed=11):
    g = torch.Generator(device=DEV).manual_seed(seed)

    def rn(*s):
        return torch.randn(*s, device=DEV, generator=g)

    q = torch.nn.functional.normalize(rn(B, T, H, D), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(rn(B, T, H, D), dim=-1).bfloat16()
    v = rn(B, T, H, D).bfloat16()
    d_out = rn(B, T, H, D).bfloat16()
    beta = torch.sigmoid(rn(B, T, H))
    glog = -0.1 * torch.rand(B, T, H, device=DEV, generator=g)
    return q, k, v, beta, glog, d_out


def _cut(ts, sl):
    return tuple(t[sl].contiguous() for t in ts)


def test_gdn_split_sequence_forward_and_backward():
    """scan(whole) == scan(first half) followed by scan(second half, h0 = state after the first), outputs, final
    state and every gradient (the state gradient handed back the same way)."""
    q, k, v, beta, glog, d_out = _gdn_full()
    B, T, H, D = q.shape
    half = T // 2
    zeros = torch.zeros(B, H, D, D, device=DEV)
    out, hT = ops.gated_delta_scan(q, k, v, beta, glog, 64, gate_is_log=True, h0=zeros, return_final_state=True)
    g = ops.gated_delta_scan_backward(q, k, v, beta, glog, d_out, 64, gate_is_log=True, h0=zeros)
    a = _cut((q, k, v, beta, glog, d_out), (slice(None), slice(0, half)))
    b = _cut((q, k, v, beta, glog, d_out), (slice(None), slice(half, T)))
    out_a, h_mid = ops.gated_delta_scan(*a[:5], 64, gate_is_log=True, h0=zeros, return_final_state=True)
    out_b, hT_b = ops.gated_delta_scan(*b[:5], 64, gate_is_log=True, h0=h_mid, return_final_state=True)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(out[:, :half], out_a) and torch.equal(out[:, half:], out_b)
    assert torch.equal(hT, hT_b)
    g_b = ops.gated_delta_scan_backward(*b, 64, gate_is_log=True, h0=h_mid)
    g_a = ops.gated_delta_scan_backward(*a, 64, gate_is_log=True, h0=zeros, d_final_state=g_b["dh0"])
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for name in ("dq", "dk", "dv", "dbeta", "dgate"):
        assert torch.equal(g[name][:, :half], g_a[name]), name
        assert torch.equal(g[name][:, half:], g_b[name]), name
    assert torch.equal(g["dh0"], g_a["dh0"])


def test_gdn_batch_rows_are_independent():
    q, k, v, beta, glog, d_out = _gdn_full(seed=12)
    out = ops.gated_delta_scan(q, k, v, beta, glog, 64, gate_is_log=True)
    g = ops.gated_delta_scan_backward(q, k, v, beta, glog, d_out, 64, gate_is_log=True)
    for b in (0, 5):
        one = _cut((q, k, v, beta, glog, d_out), slice(b, b + 1))
        out1 = ops.gated_delta_scan(*one[:5], 64, gate_is_log=True)
        g1 = ops.gated_delta_scan_backward(*one, 64, gate_is_log=True)
        torch.cuda.synchronize()
        assert torch.equal(out[b:b + 1], out1)
        for name in ("dq", "dk", "dv", "dbeta", "dgate"):
            assert torch.equal(g[name][b:b + 1], g1[name]), name
    assert ops.device_status() == 0


def test_gdn_saved_forward_and_staging_variants():
    """Backward from the forward's saved intermediates == recomputing backward; TMA staging == cp.async staging."""
    q, k, v, beta, glog, d_out = _gdn_full(seed=13)
    g = ops.gated_delta_scan_backward(q, k, v, beta, glog, d_out, 64, gate_is_log=True)
    out = ops.gated_delta_scan(q, k, v, beta, glog, 64, gate_is_log=True, save_for_backward=True)
    g_s = ops.gated_delta_scan_backward(q, k, v, beta, glog, d_out, 64, gate_is_log=True, use_saved=True)
    out_n = ops.gated_delta_scan(q, k, v, beta, glog, 64, gate_is_log=True, flags=_lib.MXB_GDN_NO_TMA)
    g_n = ops.gated_delta_scan_backward(q, k, v, beta, glog, d_out, 64, gate_is_log=True, flags=_lib.MXB_GDN_NO_TMA)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(out, out_n)
    for name in ("dq", "dk", "dv", "dbeta", "dgate"):
        assert torch.equal(g[name], g_s[name]), name
        assert torch.equal(g[name], g_n[name]), name
    assert all(bool(torch.isfinite(t.float()).all()) for t in (out, g["dq"], g["dk"], g["dv"], g["dbeta"], g["dgate"]))


def test_gdn_decode_kernels_agree_and_match_one_step_scan():
    """256 sequences x 16 heads: the streaming decode kernel and the register kernel give the same step; a
    one-token scan from the same state gives the same output and state (fp32 I/O; summation orders differ: 1e-5)."""
    N, H, D = 256, 16, 128
    g = torch.Generator(device=DEV).manual_seed(21)

    def rn(*s):
        return torch.randn(*s, device=DEV, generator=g)

    state = 0.1 * rn(N, H, D, D)
    q = torch.nn.functional.normalize(rn(N, H, D), dim=-1)
    k = torch.nn.functional.normalize(rn(N, H, D), dim=-1)
    v = rn(N, H, D)
    beta = torch.sigmoid(rn(N, H))
    glog = -0.1 * torch.rand(N, H, device=DEV, generator=g)
    s1, s2 = state.clone(), state.clone()
    o1 = ops.gated_delta_decode_step(s1, q, k, v, beta, glog, gate_is_log=True)
    o2 = ops.gated_delta_decode_step(s2, q, k, v, beta, glog, gate_is_log=True, flags=_lib.MXB_GDN_DECODE_REGISTER_KERNEL)
    o3, s3 = ops.gated_delta_scan(q[:, None], k[:, None], v[:, None], beta[:, None], glog[:, None], 64, gate_is_log=True,
                                  h0=state, return_final_state=True)
    torch.cuda.synchronize()

    def close(x, y, tol):
        return float((x.double() - y.double()).abs().max()) <= tol * max(1.0, float(y.double().abs().max()))

    assert close(o1, o2, 1e-5) and close(s1, s2, 1e-5)
    assert close(o1, o3[:, 0], 1e-4) and close(s1, s3, 1e-4)


def test_gdn_config1_sub_batch_against_oracle():
    """One sequence of the benchmark configuration (T=4096, H=16, d=128, chunk 64, bf16 I/O) against the float64 oracle
    in its chunked form (itself checked against the naive recurrence on the small shapes): outputs, final state and
    every gradient within 2e-2."""
    a = inputs.gdn_inputs(1, 4096, 16, 128, 128, seed=1, io_dtype=torch.bfloat16, with_grad_out=True)
    f = {k: v.double() for k, v in a.items()}
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], f["g"], f["d_out"], gate_is_log=True, chunk_size=64)
    dev = {k: v.to(DEV).contiguous() for k, v in a.items()}
    o, s = ops.gated_delta_scan(dev["q"], dev["k"], dev["v"], dev["beta"], dev["g"], 64, gate_is_log=True,
                                return_final_state=True)
    got = ops.gated_delta_scan_backward(dev["q"], dev["k"], dev["v"], dev["beta"], dev["g"], dev["d_out"], 64,
                                        gate_is_log=True)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(o, want["out"], 2e-2, "out")
    assert_close(s, want["state"], 2e-2, "final_state")
    for name in ("dq", "dk", "dv", "dbeta", "dgate"):
        assert_close(got[name], want[name], 2e-2, name)


def _m3_full(B=8, T=4096, NH=32, P=64, N=128, seed=31):
    g = torch.Generator(device=DEV).manual_seed(seed)
    D = NH * P
    x = torch.randn(B, T, D, device=DEV, generator=g).bfloat16()
    b = torch.randn(B, T, 1, N, device=DEV, generator=g).bfloat16()
    c = torch.randn(B, T, 1, N, device=DEV, generator=g).bfloat16()
    dt_raw = -2.0 + 0.5 * torch.randn(B, T, NH, device=DEV, generator=g)
    a_log = math.log(16.0) * torch.rand(NH, device=DEV, generator=g)
    theta = (2.0 * torch.rand(B, T, NH, device=DEV, generator=g) - 1.0) * math.pi
    lam = torch.randn(B, T, NH, device=DEV, generator=g)
    dy = torch.randn(B, T, D, device=DEV, generator=g).bfloat16()
    return (x, dt_raw, lam, theta, a_log, b, c), dy


M3_GRADS = ("dx", "ddt", "dlambda", "dtheta", "da_log", "db", "dc")


def test_mamba3_saved_forward_staging_variants_and_batch_rows():
    args, dy = _m3_full()
    NH = 32
    y = ops.mamba3_selective_scan(*args, nheads=NH)
    g = ops.mamba3_selective_scan_backward(*args, dy, nheads=NH)
    y_s = ops.mamba3_selective_scan(*args, nheads=NH, save_for_backward=True)
    g_s = ops.mamba3_selective_scan_backward(*args, dy, nheads=NH, use_saved=True)
    y_n = ops.mamba3_selective_scan(*args, nheads=NH, flags=_lib.MXB_MAMBA3_NO_TMA)
    g_n = ops.mamba3_selective_scan_backward(*args, dy, nheads=NH, flags=_lib.MXB_MAMBA3_NO_TMA)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(y, y_s) and torch.equal(y, y_n)
    for name in M3_GRADS:
        assert torch.equal(g[name], g_s[name]), name
        assert torch.equal(g[name], g_n[name]), name
        assert bool(torch.isfinite(g[name].float()).all()), name
    # one batch row alone: everything but da_log (a sum over the batch) is that row of the full result
    bsel = 3
    one = tuple(t if t.dim() == 1 else t[bsel:bsel + 1].contiguous() for t in args)
    y1 = ops.mamba3_selective_scan(*one, nheads=NH)
    g1 = ops.mamba3_selective_scan_backward(*one, dy[bsel:bsel + 1].contiguous(), nheads=NH)
    torch.cuda.synchronize()
    assert torch.equal(y[bsel:bsel + 1], y1)
    for name in M3_GRADS:
        if name != "da_log":
            assert torch.equal(g[name][bsel:bsel + 1], g1[name]), name


def test_mamba3_full_length_two_heads_against_oracle():
    """T=4096 (64 chunks: the state chain and the wrapped angle at the benchmark length), two heads of 64 channels,
    d_state 128, bf16 I/O, against the float64 oracle on the bf16-rounded inputs: output and every gradient within 2e-2."""
    from oracle import mamba3
    B, T, H, P, N = 1, 4096, 2, 64, 128
    args = ("x", "dt_raw", "lambda_raw", "theta", "a_log", "b", "c")
    a = inputs.mamba3_inputs(B, T, H, P, N, G=1, seed=6, io_dtype=torch.bfloat16, per_head=True)
    full = inputs.mamba3_expand_per_head(a)
    y_ref, want = mamba3.scan_vjp(*(full[k].double() for k in args), a["dy"].double())
    want = dict(want)
    want["ddt"] = want["ddt"].reshape(B, T, H, P).sum(-1)
    want["dlambda"] = want["dlambda"].reshape(B, T, H, P).sum(-1)
    want["dtheta"] = want["dtheta"].reshape(B, T, H, P, N // 2).sum((-1, -2))
    want["da_log"] = want["da_log"].reshape(H, P, N).sum((-1, -2))
    dev = [a[k].to(DEV).contiguous() for k in args]
    y = ops.mamba3_selective_scan(*dev, nheads=H)
    got = ops.mamba3_selective_scan_backward(*dev, a["dy"].to(DEV).contiguous(), nheads=H)
    torch.cuda.synchronize()
    assert_close(y, y_ref, 2e-2, "y")
    for name in M3_GRADS:
        assert_close(got[name], want[name], 2e-2, name)


def test_mamba3_full_size_chunked_against_recurrent_kernels():
    """Config-3 size: the chunked tensor-core kernels against the recurrent CTA-per-head kernels (a different
    algorithm for the same mathematics, itself checked against the oracle on small shapes), 2e-2."""
    args, dy = _m3_full(seed=32)
    NH = 32
    y = ops.mamba3_selective_scan(*args, nheads=NH)
    g = ops.mamba3_selective_scan_backward(*args, dy, nheads=NH)
    torch.cuda.synchronize()
    assert ops.device_status() == 0  # (the status word leads the chunked kernels' workspace only)
    y_r = ops.mamba3_selective_scan(*args, nheads=NH, flags=_lib.MXB_MAMBA3_RECURRENT_KERNELS)
    g_r = ops.mamba3_selective_scan_backward(*args, dy, nheads=NH, flags=_lib.MXB_MAMBA3_RECURRENT_KERNELS)
    torch.cuda.synchronize()
    assert_close(y, y_r.double(), 2e-2, "y")
    for name in M3_GRADS:
        assert_close(g[name], g_r[name].double(), 2e-2, name)


def test_gdn_float32_tensors_on_tensor_core_kernels_full_size():
    """MXB_GDN_F32_IO_BF16_OPERANDS at the benchmark size: float32 tensors give exactly what the bf16 entry gives on
    the rounded tensors (outputs and every gradient, widened), through the saving forward and the saved backward."""
    flag = _lib.MXB_GDN_F32_IO_BF16_OPERANDS
    q, k, v, beta, glog, d_out = _gdn_full(B=4)
    want_o = ops.gated_delta_scan(q, k, v, beta, glog, 64, gate_is_log=True)
    want = ops.gated_delta_scan_backward(q, k, v, beta, glog, d_out, 64, gate_is_log=True)
    qf, kf, vf, dof = (t.float() for t in (q, k, v, d_out))  # exactly representable: rounding them back is the identity
    got_o = ops.gated_delta_scan(qf, kf, vf, beta, glog, 64, gate_is_log=True, flags=flag, save_for_backward=True)
    got = ops.gated_delta_scan_backward(qf, kf, vf, beta, glog, dof, 64, gate_is_log=True, flags=flag, use_saved=True)
    assert got_o.dtype == torch.float32 and torch.equal(got_o, want_o.float())
    for name in ("dq", "dk", "dv", "dbeta", "dgate"):
        assert torch.equal(got[name], want[name].float()), name


def test_mamba3_channel_kernels_window_parallel_against_serial_walk_long():
    """The reference's per-channel layout at T=4096 (256 windows), d_state 16, two groups: the window-parallel kernels
    against the serial walk of the same recurrence (different summation orders: 1e-4), and bit-identical repeats."""
    from oracle import inputs as oin
    B, T, D, N, G = 2, 4096, 256, 16, 2
    a = oin.mamba3_inputs(B, T, D, 1, N, G=G, seed=5, per_head=False)
    names = ("x", "dt_raw", "lambda_raw", "theta", "a_log", "b", "c")
    dev = [a[n].to(DEV).contiguous() for n in names]
    dy = a["dy"].to(DEV).contiguous()
    ys = ops.mamba3_selective_scan(*dev, flags=_lib.MXB_MAMBA3_SERIAL_WALK)
    yw = ops.mamba3_selective_scan(*dev, flags=_lib.MXB_MAMBA3_WINDOW_PARALLEL)
    assert_close(yw, ys.double(), 1e-4, "y")
    gs = ops.mamba3_selective_scan_backward(*dev, dy, flags=_lib.MXB_MAMBA3_SERIAL_WALK)
    gw = ops.mamba3_selective_scan_backward(*dev, dy, flags=_lib.MXB_MAMBA3_WINDOW_PARALLEL)
    gw = {k2: v2.clone() for k2, v2 in gw.items()}
    for name in ("dx", "ddt", "dlambda", "dtheta", "da_log", "db", "dc"):
        assert_close(gw[name], gs[name].double(), 1e-4, name)
    again = ops.mamba3_selective_scan_backward(*dev, dy, flags=_lib.MXB_MAMBA3_WINDOW_PARALLEL)
    for name in gw:
        assert torch.equal(gw[name], again[name]), name
