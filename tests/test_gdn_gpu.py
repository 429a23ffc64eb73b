"""Parity of the CUDA gated-delta kernels (through the C ABI) with the CPU oracle."""
import json
import os

import numpy as np
import pytest
import torch

import mixlab_b200
from mixlab_b200 import ops
from oracle import gdn, inputs
from tests.util import assert_close

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"
TOL_F32 = 1e-4   # fp32 I/O
TOL_BF16 = 2e-2  # bf16 I/O, fp32 state


def _dev(t):
    return None if t is None else t.to(DEV).contiguous()


def _oracle_fwd(a, chunk, h0=None):
    f = {k: v.double() for k, v in a.items() if torch.is_tensor(v)}
    return gdn.scan_chunked(f["q"], f["k"], f["v"], f["beta"], torch.exp(f["g"]), chunk,
                            None if h0 is None else h0.double())


@pytest.mark.parametrize("shape", [
    (2, 256, 4, 64, 64, 64),     # benchmark config 0
    (2, 97, 3, 8, 12, 64),       # the reference test's ragged shape
    (1, 1, 1, 4, 4, 64),         # a single token
    (1, 63, 2, 16, 8, 64), (1, 65, 2, 16, 8, 64), (1, 130, 1, 32, 20, 16),
    (1, 200, 2, 128, 128, 64),
    (1, 50, 2, 8, 8, 0),         # token-by-token recurrence
])
@pytest.mark.parametrize("gate_is_log", [True, False])
def test_forward_fp32(shape, gate_is_log):
    B, T, H, K, V, C = shape
    a = inputs.gdn_inputs(B, T, H, K, V, seed=0, with_h0=True)
    want_o, want_s = _oracle_fwd(a, C, a["h0"])
    gate = a["g"] if gate_is_log else torch.exp(a["g"])
    o, s = ops.gated_delta_scan(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(gate), C,
                                gate_is_log=gate_is_log, h0=_dev(a["h0"]), return_final_state=True)
    assert_close(o, want_o, TOL_F32, "out")
    assert_close(s, want_s, TOL_F32, "final_state")


def test_forward_config0_zero_state():
    """B=2,T=256,H=4,d=64, chunk 64, seed 0, zero initial state (benchmark config 0)."""
    a = inputs.gdn_inputs(2, 256, 4, 64, 64, seed=0)
    want_o, want_s = _oracle_fwd(a, 64)
    o, s = ops.gated_delta_scan(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]), 64,
                                gate_is_log=True, return_final_state=True)
    assert o.shape == (2, 256, 4, 64) and s.shape == (2, 4, 64, 64)
    assert_close(o, want_o, TOL_F32, "out")
    assert_close(s, want_s, TOL_F32, "final_state")


@pytest.mark.parametrize("shape", [
    (2, 256, 4, 64, 64, 64), (2, 97, 3, 8, 12, 64), (1, 130, 2, 32, 20, 16), (1, 70, 1, 128, 128, 64),
    (1, 40, 2, 8, 8, 0),
])
@pytest.mark.parametrize("gate_is_log", [True, False])
def test_backward_fp32(shape, gate_is_log):
    B, T, H, K, V, C = shape
    a = inputs.gdn_inputs(B, T, H, K, V, seed=1, with_grad_out=True, with_h0=True)
    f = {k: v.double() for k, v in a.items()}
    gate64 = f["g"] if gate_is_log else torch.exp(f["g"])
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], gate64, f["d_out"], f["d_state"], f["h0"],
                          gate_is_log=gate_is_log)
    gate = a["g"] if gate_is_log else torch.exp(a["g"])
    got = ops.gated_delta_scan_backward(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(gate),
                                        _dev(a["d_out"]), C, gate_is_log=gate_is_log, h0=_dev(a["h0"]),
                                        d_final_state=_dev(a["d_state"]))
    for name in ("dq", "dk", "dv", "dbeta", "dgate", "dh0"):
        assert_close(got[name], want[name], TOL_F32, name)


def test_reference_golden_vectors():
    """The reference's own scalar/torch scan outputs (tests/golden) through the CUDA path."""
    with open(os.path.join(G, "gdn_scalar_reference.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        B, T, H, K, V = (c[x] for x in ("B", "T", "H", "Dk", "Dv"))
        t = lambda key, *s: torch.tensor(c[key], dtype=torch.float32).reshape(*s)
        for chunk in (0, 64):
            o = ops.gated_delta_scan(_dev(t("q", B, T, H, K)), _dev(t("k", B, T, H, K)), _dev(t("v", B, T, H, V)),
                                     _dev(t("beta", B, T, H)), _dev(t("gate", B, T, H)), chunk)
            assert_close(o, torch.tensor(c["out"], dtype=torch.float64).reshape(B, T, H, V), TOL_F32, c["name"])
    z = np.load(os.path.join(G, "gdn_torch_recurrence.npz"))
    a = {k: torch.from_numpy(z[k]) for k in z.files}
    o = ops.gated_delta_scan(*(_dev(a[k].float()) for k in ("q", "k", "v", "beta", "gate")), 64)
    assert_close(o, a["out"], TOL_F32, "torch_recurrence")


def test_go_test_inputs_chunked_matches_naive():
    """gpu/gated_delta_scan_test.go:174-263 on the CUDA path: chunk 64 vs chunk 0, tol 1e-4."""
    z = np.load(os.path.join(G, "gdn_go_test_inputs.npz"))
    a = [_dev(torch.from_numpy(z[k]).float()) for k in ("q", "k", "v", "beta", "gate")]
    o0 = ops.gated_delta_scan(*a, 0)
    o64 = ops.gated_delta_scan(*a, 64)
    assert (o0 - o64).abs().max().item() <= 1e-4


@pytest.mark.parametrize("shape", [(1, 256, 2, 128, 128, 64), (2, 100, 2, 64, 64, 64)])
def test_forward_backward_bf16_io(shape):
    """bf16 q,k,v,dO with fp32 state: 2e-2 against the float64 oracle on the bf16-rounded inputs."""
    B, T, H, K, V, C = shape
    a = inputs.gdn_inputs(B, T, H, K, V, seed=1, io_dtype=torch.bfloat16, with_grad_out=True)
    f = {k: v.double() for k, v in a.items()}
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], f["g"], f["d_out"], gate_is_log=True)
    o, s = ops.gated_delta_scan(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]), C,
                                gate_is_log=True, return_final_state=True)
    assert o.dtype == torch.bfloat16
    assert_close(o, want["out"], TOL_BF16, "out")
    assert_close(s, want["state"], TOL_BF16, "final_state")
    got = ops.gated_delta_scan_backward(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]),
                                        _dev(a["d_out"]), C, gate_is_log=True)
    for name in ("dq", "dk", "dv", "dbeta", "dgate"):
        assert_close(got[name], want[name], TOL_BF16, name)


def test_decode_steps():
    """Recurrent decode: parity after 1, 16 and 64 steps on 4 sequences (config 2 dims)."""
    N, H, K, V, steps = 4, 16, 128, 128, 64
    a = inputs.gdn_decode_inputs(N, H, K, V, steps, seed=2, io_dtype=torch.bfloat16)
    st_ref = a["state"].double()
    st = _dev(a["state"].clone())
    for t in range(steps):
        o_ref, st_ref = gdn.decode_step(st_ref, a["q"][t].double(), a["k"][t].double(), a["v"][t].double(),
                                        a["beta"][t].double(), torch.exp(a["g"][t].double()))
        o = ops.gated_delta_decode_step(st, _dev(a["q"][t]), _dev(a["k"][t]), _dev(a["v"][t]), _dev(a["beta"][t]),
                                        _dev(a["g"][t]), gate_is_log=True)
        if t + 1 in (1, 16, 64):
            assert_close(o, o_ref, TOL_BF16, f"out@{t + 1}")
            assert_close(st, st_ref, 1e-4, f"state@{t + 1}")


def test_decode_1024_steps():
    """Recurrent decode: the state and the output after 1024 steps on 4 sequences (config 2 dims) still match the
    float64 recurrence (fp32 state, bf16 tokens)."""
    N, H, K, V, steps = 4, 16, 128, 128, 1024
    a = inputs.gdn_decode_inputs(N, H, K, V, steps, seed=22, io_dtype=torch.bfloat16)
    st_ref = a["state"].double()
    st = _dev(a["state"].clone())
    q, k, v, beta, g = (_dev(a[n]) for n in ("q", "k", "v", "beta", "g"))
    for t in range(steps):
        o_ref, st_ref = gdn.decode_step(st_ref, a["q"][t].double(), a["k"][t].double(), a["v"][t].double(),
                                        a["beta"][t].double(), torch.exp(a["g"][t].double()))
        o = ops.gated_delta_decode_step(st, q[t], k[t], v[t], beta[t], g[t], gate_is_log=True)
        if t + 1 in (256, 1024):
            assert_close(o, o_ref, TOL_BF16, f"out@{t + 1}")
            assert_close(st, st_ref, 1e-4, f"state@{t + 1}")


@pytest.mark.parametrize("dims", [(3, 2, 64, 64), (2, 3, 8, 12), (1, 1, 200, 256), (2, 2, 40, 132)])
def test_decode_fp32_shapes(dims):
    N, H, K, V = dims
    a = inputs.gdn_decode_inputs(N, H, K, V, 3, seed=5, io_dtype=torch.float32)
    st_ref = a["state"].double()
    st = _dev(a["state"].clone())
    for t in range(3):
        gate = torch.exp(a["g"][t])
        o_ref, st_ref = gdn.decode_step(st_ref, a["q"][t].double(), a["k"][t].double(), a["v"][t].double(),
                                        a["beta"][t].double(), gate.double())
        o = ops.gated_delta_decode_step(st, _dev(a["q"][t]), _dev(a["k"][t]), _dev(a["v"][t]), _dev(a["beta"][t]),
                                        _dev(gate))
        assert_close(o, o_ref, TOL_F32, "out")
    assert_close(st, st_ref, TOL_F32, "state")


def test_decode_equals_scan():
    """T decode steps from a zero state reproduce the scan output (same recurrence)."""
    a = inputs.gdn_inputs(2, 24, 2, 64, 64, seed=4)
    o_scan, s_scan = ops.gated_delta_scan(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]), 64,
                                          gate_is_log=True, return_final_state=True)
    st = torch.zeros(2, 2, 64, 64, device=DEV)
    for t in range(24):
        o = ops.gated_delta_decode_step(st, _dev(a["q"][:, t]), _dev(a["k"][:, t]), _dev(a["v"][:, t]),
                                        _dev(a["beta"][:, t]), _dev(a["g"][:, t]), gate_is_log=True)
        assert_close(o, o_scan[:, t], TOL_F32, f"o[{t}]")
    assert_close(st, s_scan, TOL_F32, "state")


@pytest.mark.parametrize("B,H,split", [(1, 2, None), (3, 2, None), (4, 2, None), (3, 4, "2"), (1, 4, "4"), (2, 6, "3")])
def test_host_buffer_entry_point(B, H, split, monkeypatch):
    """mxb_host_gdn: host tensors in, host tensors out, forward + backward (slices are pipelined through two device
    slots, so more than two slices exercise slot reuse; with a head split a slice is a group of heads of one sequence,
    moved by strided copies)."""
    import ctypes as C
    lib = mixlab_b200.lib()
    if split is not None:
        monkeypatch.setenv("MXB_HOST_HEAD_SPLIT", split)
    T, K, V = 100, 32, 32
    a = inputs.gdn_inputs(B, T, H, K, V, seed=6, with_grad_out=True)
    f = {k: v.double() for k, v in a.items()}
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], f["g"], f["d_out"], gate_is_log=True)
    ctx = C.c_void_p()
    assert lib.mxb_host_ctx_create(0, 64 << 20, C.byref(ctx)) == 0
    try:
        d = mixlab_b200.GdnDesc(B, T, H, K, V, 64, mixlab_b200.MXB_F32, 1, 0)
        out = torch.empty_like(a["v"])
        dq, dk, dv = torch.empty_like(a["q"]), torch.empty_like(a["k"]), torch.empty_like(a["v"])
        db, dg = torch.empty_like(a["beta"]), torch.empty_like(a["g"])
        p = lambda t: C.c_void_p(t.data_ptr())
        st = lib.mxb_host_gdn(ctx, C.byref(d), p(a["q"]), p(a["k"]), p(a["v"]), p(a["beta"]), p(a["g"]), p(out),
                              p(a["d_out"]), p(dq), p(dk), p(dv), p(db), p(dg))
        assert st == 0
    finally:
        lib.mxb_host_ctx_destroy(ctx)
    assert_close(out, want["out"], TOL_F32, "out")
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv), ("dbeta", db), ("dgate", dg)):
        assert_close(t, want[name], TOL_F32, name)


def test_launch_counter_moves():
    lib = mixlab_b200.lib()
    n0 = lib.mxb_launch_count()
    a = inputs.gdn_inputs(1, 8, 1, 8, 8, seed=0)
    ops.gated_delta_scan(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]), 64, gate_is_log=True)
    torch.cuda.synchronize()
    assert lib.mxb_launch_count() >= n0 + 2


# ---------------------------------------------------------------- tensor-core path (bf16, d=128, chunk 64)
@pytest.mark.parametrize("shape", [(1, 64, 1), (1, 200, 2), (2, 512, 3), (1, 1, 1), (1, 65, 1)])
@pytest.mark.parametrize("with_h0", [False, True])
def test_tensor_core_forward(shape, with_h0):
    """tcgen05 forward vs the float64 oracle on the bf16-rounded inputs, and vs the fp32 CUDA-core kernels."""
    from mixlab_b200 import _lib
    B, T, H = shape
    a = inputs.gdn_inputs(B, T, H, 128, 128, seed=11, io_dtype=torch.bfloat16, with_h0=with_h0)
    h0 = a.get("h0")
    want_o, want_s = _oracle_fwd(a, 64, h0)
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]), 64)
    o, s = ops.gated_delta_scan(*args, gate_is_log=True, h0=_dev(h0), return_final_state=True)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(o, want_o, TOL_BF16, "out")
    assert_close(s, want_s, TOL_BF16, "final_state")
    o32, s32 = ops.gated_delta_scan(*args, gate_is_log=True, h0=_dev(h0), return_final_state=True,
                                    flags=_lib.MXB_GDN_FORCE_FP32_PATH)
    assert_close(o, o32.float(), TOL_BF16, "out vs fp32 kernels")
    assert_close(s, s32, TOL_BF16, "state vs fp32 kernels")


def test_tensor_core_forward_multiplicative_gate():
    a = inputs.gdn_inputs(1, 130, 2, 128, 128, seed=12, io_dtype=torch.bfloat16)
    want_o, _ = _oracle_fwd(a, 64)
    o = ops.gated_delta_scan(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(torch.exp(a["g"])), 64)
    assert_close(o, want_o, TOL_BF16, "out")


@pytest.mark.parametrize("shape", [(1, 64, 1), (1, 200, 2), (2, 320, 2), (1, 1, 1)])
@pytest.mark.parametrize("with_h0", [False, True])
@pytest.mark.parametrize("gate_is_log", [True, False])
def test_tensor_core_backward(shape, with_h0, gate_is_log):
    """tcgen05 backward vs float64 autograd on the bf16-rounded inputs (2e-2 on every gradient)."""
    B, T, H = shape
    a = inputs.gdn_inputs(B, T, H, 128, 128, seed=21, io_dtype=torch.bfloat16, with_grad_out=True, with_h0=with_h0)
    f = {k: v.double() for k, v in a.items()}
    gate64 = f["g"] if gate_is_log else torch.exp(f["g"])
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], gate64, f["d_out"], f.get("d_state"), f.get("h0"),
                          gate_is_log=gate_is_log)
    gate = a["g"] if gate_is_log else torch.exp(a["g"])
    got = ops.gated_delta_scan_backward(_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(gate),
                                        _dev(a["d_out"]), 64, gate_is_log=gate_is_log, h0=_dev(a.get("h0")),
                                        d_final_state=_dev(a.get("d_state")))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    names = ["dq", "dk", "dv", "dbeta", "dgate"] + (["dh0"] if with_h0 else [])
    errs = {}
    for name in names:
        try:
            errs[name] = assert_close(got[name], want[name], TOL_BF16, name)
        except AssertionError as e:
            errs[name] = str(e)
    assert all(not isinstance(v, str) for v in errs.values()), errs


def test_tensor_core_backward_matches_fp32_kernels():
    from mixlab_b200 import _lib
    a = inputs.gdn_inputs(1, 256, 2, 128, 128, seed=22, io_dtype=torch.bfloat16, with_grad_out=True)
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]), _dev(a["d_out"]), 64)
    g_tc = ops.gated_delta_scan_backward(*args, gate_is_log=True)
    g_32 = ops.gated_delta_scan_backward(*args, gate_is_log=True, flags=_lib.MXB_GDN_BWD_FP32_KERNELS)
    for name in ("dq", "dk", "dv", "dbeta", "dgate"):
        assert_close(g_tc[name], g_32[name].float(), TOL_BF16, name)


@pytest.mark.parametrize("case", [(2, 200, 2, 128, 128, torch.bfloat16), (1, 130, 2, 32, 20, torch.float32)])
def test_backward_from_saved_forward(case):
    """Forward with save_for_backward + backward with use_saved == backward with its own recompute."""
    B, T, H, K, V, io = case
    a = inputs.gdn_inputs(B, T, H, K, V, seed=31, io_dtype=io, with_grad_out=True, with_h0=True)
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]))
    kw = dict(gate_is_log=True, h0=_dev(a["h0"]))
    ref = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), 64, d_final_state=_dev(a["d_state"]), **kw)
    o_plain = ops.gated_delta_scan(*args, 64, **kw)
    o = ops.gated_delta_scan(*args, 64, save_for_backward=True, **kw)
    got = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), 64, d_final_state=_dev(a["d_state"]),
                                        use_saved=True, **kw)
    assert torch.equal(o, o_plain)
    for name in ("dq", "dk", "dv", "dbeta", "dgate", "dh0"):
        assert torch.equal(got[name], ref[name]), name


@pytest.mark.parametrize("dims", [(40, 16, 128, 128, torch.bfloat16), (10, 3, 64, 128, torch.float32),
                                  (150, 4, 128, 128, torch.float32)])
def test_decode_bulk_pipeline(dims):
    """The bulk-copy pipelined decode kernel with several tiles per CTA, against the oracle and
    against the register-resident kernel."""
    from mixlab_b200 import _lib
    N, H, K, V, io = dims
    a = inputs.gdn_decode_inputs(N, H, K, V, 3, seed=7, io_dtype=io)
    st_ref = a["state"].double()
    st = _dev(a["state"].clone())
    st_reg = _dev(a["state"].clone())
    tol = TOL_F32 if io == torch.float32 else TOL_BF16
    for t in range(3):
        o_ref, st_ref = gdn.decode_step(st_ref, a["q"][t].double(), a["k"][t].double(), a["v"][t].double(),
                                        a["beta"][t].double(), torch.exp(a["g"][t].double()))
        args = (_dev(a["q"][t]), _dev(a["k"][t]), _dev(a["v"][t]), _dev(a["beta"][t]), _dev(a["g"][t]))
        o = ops.gated_delta_decode_step(st, *args, gate_is_log=True)
        o_reg = ops.gated_delta_decode_step(st_reg, *args, gate_is_log=True, flags=_lib.MXB_GDN_DECODE_REGISTER_KERNEL)
        assert_close(o, o_ref, tol, f"out@{t}")
        assert_close(o, o_reg.double(), tol, f"out vs register kernel@{t}")
    assert_close(st, st_ref, TOL_F32, "state")
    assert_close(st, st_reg.double(), 1e-5, "state vs register kernel")


@pytest.mark.parametrize("T", [64, 200, 513])
def test_tensor_core_tma_matches_cp_async_staging(T):
    """The prep kernel fed by TMA tensor copies (128-byte swizzle, zero-filled ragged tail) gives the same bits as
    the cp.async staging of the same tiles."""
    from mixlab_b200 import _lib
    a = inputs.gdn_inputs(2, T, 2, 128, 128, seed=41, io_dtype=torch.bfloat16, with_grad_out=True)
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]))
    o1, s1 = ops.gated_delta_scan(*args, 64, gate_is_log=True, return_final_state=True)
    o2, s2 = ops.gated_delta_scan(*args, 64, gate_is_log=True, return_final_state=True, flags=_lib.MXB_GDN_NO_TMA)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    g1 = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), 64, gate_is_log=True)
    g2 = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), 64, gate_is_log=True, flags=_lib.MXB_GDN_NO_TMA)
    for name in ("dq", "dk", "dv", "dbeta", "dgate"):
        assert torch.equal(g1[name], g2[name]), name


# ---------------------------------------------------------------- numeric guards, chunk sizes, wide values
def _guard_case(kind, B, T, H, K, V, io, seed=51):
    """Inputs on which the reference's guards change the result (gpu/ir.cpp:35-37): gates at and below the floor of
    1e-30 (multiplicative form) or log decays whose in-chunk cumulative sum passes -80 / falls below log(1e-30)."""
    a = inputs.gdn_inputs(B, T, H, K, V, seed=seed, io_dtype=io, with_grad_out=True, with_h0=True)
    g = a["g"].clone()
    if kind == "tiny_gates":      # multiplicative gate with exact zeros and values around the floor
        gate = torch.exp(g)
        flat = gate.view(-1)
        for off, val in ((5, 0.0), (17, 1e-38), (29, 1e-31), (43, 1e-29)):
            flat[off::97] = val
        return a, gate, False
    if kind == "steep":           # -3 per token: the in-chunk cumulative sum passes -80 after 27 tokens
        return a, torch.full_like(g, -3.0), True
    if kind == "abyss":           # single log decays below log(1e-30) = -69.08
        flat = g.view(-1)
        flat[7::53] = -200.0
        return a, g, True
    raise ValueError(kind)


def _check_guard_case(kind, shape, io, tol, flags=0, chunk=64):
    B, T, H, K, V = shape
    a, gate, is_log = _guard_case(kind, B, T, H, K, V, io)
    f = {k: v.double() for k, v in a.items()}
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], gate.double(), f["d_out"], f["d_state"], f["h0"],
                          gate_is_log=is_log, chunk_size=64)
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(gate))
    o, s = ops.gated_delta_scan(*args, chunk, gate_is_log=is_log, h0=_dev(a["h0"]), return_final_state=True, flags=flags)
    got = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), chunk, gate_is_log=is_log, h0=_dev(a["h0"]),
                                        d_final_state=_dev(a["d_state"]), flags=flags)
    torch.cuda.synchronize()
    assert_close(o, want["out"], tol, f"{kind}: out")
    assert_close(s, want["state"], tol, f"{kind}: final_state")
    for name in ("dq", "dk", "dv", "dbeta", "dh0"):
        assert_close(got[name], want[name], tol, f"{kind}: {name}")
    if is_log:
        assert_close(got["dgate"], want["dgate"], tol, f"{kind}: dgate")
    else:
        # d/d(gate) = d/d(log gate) / gate: next to a gate of 1e-29 the division turns the rounding error of the
        # log-gate gradient (a reverse cumulative sum of O(1) terms, in fp32 here as in the reference) into 1e22, so
        # the two are compared as gradients with respect to log gate, where the tolerance means something
        gd = _dev(gate).double()
        assert_close(got["dgate"].double() * gd, want["dgate"].to(DEV) * gd, tol, f"{kind}: dgate * gate")
    return a, gate, is_log, got


@pytest.mark.parametrize("kind", ["tiny_gates", "steep", "abyss"])
@pytest.mark.parametrize("shape", [(2, 130, 2, 16, 24), (1, 200, 2, 64, 64)])
def test_numeric_guards_fp32(kind, shape):
    """fp32 kernels on the inputs the gate floor and the exponent clamp exist for, against the float64 oracle of the
    chunked form (which carries the same guards): outputs, final state, every gradient, all finite."""
    a, gate, is_log, got = _check_guard_case(kind, shape, torch.float32, TOL_F32)
    if kind == "tiny_gates":  # the gradient with respect to a gate below the floor is exactly zero (clamp)
        below = _dev(gate) < 1e-30
        assert below.any() and (got["dgate"][below] == 0).all()


@pytest.mark.parametrize("kind", ["tiny_gates", "steep", "abyss"])
def test_numeric_guards_tensor_core(kind):
    """The same inputs through the tcgen05 kernels (bf16 I/O, d = 128, chunk 64) at 2e-2."""
    _check_guard_case(kind, (1, 200, 2, 128, 128), torch.bfloat16, TOL_BF16)
    assert ops.device_status() == 0


@pytest.mark.parametrize("kind", ["tiny_gates", "abyss"])
def test_recurrence_has_no_gate_floor(kind):
    """chunk <= 1 and the decode step follow gated_delta_scan_naive (gpu/ir.cpp:2334), which applies no floor: a zero
    gate empties the state exactly.  The backward of chunk <= 1 differentiates the chunked form (its gate gradient is
    zero below the floor); all other gradients agree with the recurrence's to fp32 accuracy."""
    B, T, H, K, V = 2, 60, 2, 16, 24
    a, gate, is_log = _guard_case(kind, B, T, H, K, V, torch.float32)
    f = {k: v.double() for k, v in a.items()}
    g64 = torch.exp(gate.double()) if is_log else gate.double()
    want_o, want_s = gdn.scan_naive(f["q"], f["k"], f["v"], f["beta"], g64, f["h0"])
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(gate))
    o, s = ops.gated_delta_scan(*args, 0, gate_is_log=is_log, h0=_dev(a["h0"]), return_final_state=True)
    assert_close(o, want_o, TOL_F32, "out")
    assert_close(s, want_s, TOL_F32, "final_state")
    st = _dev(a["h0"].clone())
    for t in range(T):
        od = ops.gated_delta_decode_step(st, *(x[:, t].contiguous() for x in args), gate_is_log=is_log)
        assert_close(od, want_o[:, t], TOL_F32, f"decode out[{t}]")
    assert_close(st, want_s, TOL_F32, "decode state")
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], gate.double(), f["d_out"], f["d_state"], f["h0"],
                          gate_is_log=is_log, chunk_size=64)
    got = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), 0, gate_is_log=is_log, h0=_dev(a["h0"]),
                                        d_final_state=_dev(a["d_state"]))
    for name in ("dq", "dk", "dv", "dbeta", "dh0"):
        assert_close(got[name], want[name], TOL_F32, name)
    scale = _dev(gate).double() if not is_log else 1.0   # compared as gradients with respect to log gate
    assert_close(got["dgate"].double() * scale, want["dgate"].to(DEV) * scale, TOL_F32, "dgate")


@pytest.mark.parametrize("case", [(2, 300, 2, 32, 20, torch.float32, 0), (1, 300, 2, 128, 128, torch.bfloat16, 0),
                                  (1, 300, 2, 128, 128, torch.bfloat16, 1)])
def test_chunk_above_64_equals_chunk_64(case):
    """The reference accepts scan_chunk_size overrides above 64 (arch/blocks_gated_deltanet.go:11-17); the result does
    not depend on the chunk size and is computed with chunks of 64: same bits."""
    from mixlab_b200 import _lib
    B, T, H, K, V, io, fp32_path = case
    flags = _lib.MXB_GDN_FORCE_FP32_PATH if fp32_path else 0
    a = inputs.gdn_inputs(B, T, H, K, V, seed=61, io_dtype=io, with_grad_out=True)
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]))
    res = {}
    for chunk in (64, 128, 256):
        o, s = ops.gated_delta_scan(*args, chunk, gate_is_log=True, return_final_state=True, flags=flags)
        g = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), chunk, gate_is_log=True, flags=flags)
        res[chunk] = (o, s, g)
    for chunk in (128, 256):
        assert torch.equal(res[chunk][0], res[64][0]) and torch.equal(res[chunk][1], res[64][1])
        for name in ("dq", "dk", "dv", "dbeta", "dgate"):
            assert torch.equal(res[chunk][2][name], res[64][2][name]), name
    want_o, _ = _oracle_fwd(a, 128)
    assert_close(res[128][0], want_o, TOL_F32 if io == torch.float32 else TOL_BF16, "out vs oracle at chunk 128")


@pytest.mark.parametrize("shape", [(1, 100, 2, 16, 256, 64), (1, 70, 1, 128, 256, 64), (1, 40, 1, 64, 160, 0)])
def test_wide_values_fp32(shape):
    """Dv = 2 Dk is the reference default (effectiveGatedDeltaNetDV): values up to 256 wide on the fp32 kernels."""
    B, T, H, K, V, C = shape
    a = inputs.gdn_inputs(B, T, H, K, V, seed=71, with_grad_out=True, with_h0=True)
    f = {k: v.double() for k, v in a.items()}
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], f["g"], f["d_out"], f["d_state"], f["h0"], gate_is_log=True)
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]))
    o, s = ops.gated_delta_scan(*args, C, gate_is_log=True, h0=_dev(a["h0"]), return_final_state=True)
    assert_close(o, want["out"], TOL_F32, "out")
    assert_close(s, want["state"], TOL_F32, "final_state")
    got = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), C, gate_is_log=True, h0=_dev(a["h0"]),
                                        d_final_state=_dev(a["d_state"]))
    for name in ("dq", "dk", "dv", "dbeta", "dgate", "dh0"):
        assert_close(got[name], want[name], TOL_F32, name)


def test_front_end_rejects_mismatched_operands():
    """A k with fewer heads, a float32 k beside a bf16 q, an h0 of the wrong width: Python errors, no launch."""
    lib = mixlab_b200.lib()
    a = inputs.gdn_inputs(1, 32, 2, 16, 16, seed=0, with_grad_out=True, with_h0=True)
    d = {k: _dev(v) for k, v in a.items()}
    n0 = lib.mxb_launch_count()
    with pytest.raises(ValueError):
        ops.gated_delta_scan(d["q"], d["k"][:, :, :1].contiguous(), d["v"], d["beta"], d["g"], 64, gate_is_log=True)
    with pytest.raises(TypeError):
        ops.gated_delta_scan(d["q"].bfloat16(), d["k"], d["v"].bfloat16(), d["beta"], d["g"], 64, gate_is_log=True)
    with pytest.raises(ValueError):
        ops.gated_delta_scan(d["q"], d["k"], d["v"], d["beta"], d["g"], 64, gate_is_log=True, h0=d["h0"][..., :8].contiguous())
    with pytest.raises(ValueError):
        ops.gated_delta_scan_backward(d["q"], d["k"], d["v"], d["beta"], d["g"], d["d_out"][:, :16].contiguous(), 64,
                                      gate_is_log=True)
    with pytest.raises(RuntimeError):  # use_saved without a saving forward just before
        ops.gated_delta_scan(d["q"], d["k"], d["v"], d["beta"], d["g"], 64, gate_is_log=True)
        ops.gated_delta_scan_backward(d["q"], d["k"], d["v"], d["beta"], d["g"], d["d_out"], 64, gate_is_log=True,
                                      use_saved=True)
    torch.cuda.synchronize()
    assert lib.mxb_launch_count() - n0 <= 2  # only the one plain forward above launched anything


@pytest.mark.parametrize("dims", [(64, 64), (64, 128), (128, 64), (96, 72)])
@pytest.mark.parametrize("T", [200, 64])
def test_tensor_core_narrow_heads(dims, T):
    """Heads narrower than the 128-wide tiles run the same tcgen05 kernels (the copy engine zero-fills the missing
    columns and clips them on stores): forward and every gradient at 2e-2 against the float64 oracle, with initial
    state and final-state gradient; (64, 64) is the head size of the end-to-end training configuration, (64, 128) the
    reference's own benchmark shape (gpu/gated_delta_scan_test.go:265-277)."""
    K, V = dims
    lib = mixlab_b200.lib()
    a = inputs.gdn_inputs(2, T, 3, K, V, seed=81, io_dtype=torch.bfloat16, with_grad_out=True, with_h0=True)
    f = {k: v.double() for k, v in a.items()}
    want = gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], f["g"], f["d_out"], f["d_state"], f["h0"], gate_is_log=True)
    args = (_dev(a["q"]), _dev(a["k"]), _dev(a["v"]), _dev(a["beta"]), _dev(a["g"]))
    lib.mxb_trace_enable(1)
    o, s = ops.gated_delta_scan(*args, 64, gate_is_log=True, h0=_dev(a["h0"]), return_final_state=True)
    got = ops.gated_delta_scan_backward(*args, _dev(a["d_out"]), 64, gate_is_log=True, h0=_dev(a["h0"]),
                                        d_final_state=_dev(a["d_state"]))
    torch.cuda.synchronize()
    import ctypes as C
    buf = C.create_string_buffer(4096)
    lib.mxb_trace_summary(buf, len(buf))
    lib.mxb_trace_enable(0)
    assert b"gdn_tc_prep_kernel" in buf.value and b"gdn_tc_chunk_bwd_kernel" in buf.value, buf.value  # the tensor-core path ran
    assert ops.device_status() == 0
    assert_close(o, want["out"], TOL_BF16, "out")
    assert_close(s, want["state"], TOL_BF16, "final_state")
    for name in ("dq", "dk", "dv", "dbeta", "dgate", "dh0"):
        assert_close(got[name], want[name], TOL_BF16, name)


def test_ir_op_records_replay():
    """The records the reference's Go side emits for ops 60 and 63 (arch/ir.go:550-555, :600-602), replayed through
    mxb_ir_op_forward with device pointers in place of the names: same results as the reference-generated vectors."""
    with open(os.path.join(G, "gdn_scalar_reference.json")) as f:
        c = json.load(f)["cases"][2]
    B, T, H, K, V = (c[x] for x in ("B", "T", "H", "Dk", "Dv"))
    t = lambda key, *s: _dev(torch.tensor(c[key], dtype=torch.float32).reshape(*s))
    ins = [t("q", B, T, H, K), t("k", B, T, H, K), t("v", B, T, H, V), t("beta", B, T, H), t("gate", B, T, H)]
    want = torch.tensor(c["out"], dtype=torch.float64).reshape(B * T * H, V)
    for int_params in ([B, T, H, K, V, 64], [B, T, H, K, V, 0], [B, T, H, K, V]):   # chunked, recurrence, legacy record
        out = ops.ir_op_forward(60, ins, int_params, out_shape=(B * T * H, V))     # "out: [B*T*H, Dv]"
        assert_close(out, want, TOL_F32, f"op 60 {int_params}")
    z = np.load(os.path.join(G, "mamba3_torch_scan.npz"))
    Bm, Tm, D = z["b_x"].shape
    Gm, N = z["b_b"].shape[-2:]
    m = lambda key, *s: _dev(torch.from_numpy(z["b_" + key]).float().reshape(*s))
    ins = [m("x", Bm * Tm, D), m("dt_raw", Bm * Tm, D), m("lambda_raw", Bm * Tm, D), m("theta", Bm * Tm, D * N // 2),
           m("a_log", D, N), m("b", Bm * Tm, Gm * N), m("c", Bm * Tm, Gm * N)]
    for int_params in ([Bm, Tm, D, N, Gm], [Bm, Tm, D, N, Gm, 16]):
        y = ops.ir_op_forward(63, ins, int_params, out_shape=(Bm * Tm, D))
        assert_close(y, torch.from_numpy(z["b_y"]).reshape(Bm * Tm, D), TOL_F32, f"op 63 {int_params}")


@pytest.mark.parametrize("dims", [(2, 200, 2, 128, 128), (1, 130, 3, 64, 96)])
def test_float32_tensors_through_tensor_core_kernels(dims):
    """MXB_GDN_F32_IO_BF16_OPERANDS: float32 tensors in and out, bf16 operands inside.  The results must be
    exactly those of the bf16 entry on the rounded inputs (widened), stay within the bf16 tolerance of the oracle
    on the float32 inputs, and the saved-forward backward must agree with the recomputing one."""
    from mixlab_b200 import _lib
    B, T, H, K, V = dims
    flag = _lib.MXB_GDN_F32_IO_BF16_OPERANDS
    a = inputs.gdn_inputs(B, T, H, K, V, seed=77, io_dtype=torch.float32, with_grad_out=True, with_h0=True)
    q, k, v, beta, g, do = (_dev(a[n]) for n in ("q", "k", "v", "beta", "g", "d_out"))
    kw = dict(gate_is_log=True, h0=_dev(a["h0"]))
    out, hT = ops.gated_delta_scan(q, k, v, beta, g, 64, return_final_state=True, flags=flag, **kw)
    assert out.dtype == torch.float32
    q16, k16, v16, do16 = (t.to(torch.bfloat16) for t in (q, k, v, do))
    out16, hT16 = ops.gated_delta_scan(q16, k16, v16, beta, g, 64, return_final_state=True, **kw)
    assert torch.equal(out, out16.float()) and torch.equal(hT, hT16)
    ref_out, ref_state = _oracle_fwd(a, 64, h0=a["h0"])
    assert_close(out, ref_out, TOL_BF16, "out")
    assert_close(hT, ref_state, TOL_BF16, "hT")

    dst = _dev(a["d_state"])
    got = ops.gated_delta_scan_backward(q, k, v, beta, g, do, 64, d_final_state=dst, flags=flag, **kw)
    want = ops.gated_delta_scan_backward(q16, k16, v16, beta, g, do16, 64, d_final_state=dst, **kw)
    for name in ("dq", "dk", "dv", "dbeta", "dgate", "dh0"):
        assert got[name].dtype == torch.float32
        assert torch.equal(got[name], want[name].float()), name
    ops.gated_delta_scan(q, k, v, beta, g, 64, save_for_backward=True, flags=flag, **kw)
    again = ops.gated_delta_scan_backward(q, k, v, beta, g, do, 64, d_final_state=dst, flags=flag, use_saved=True, **kw)
    for name in ("dq", "dk", "dv", "dbeta", "dgate", "dh0"):
        assert torch.equal(again[name], got[name]), name
    # without the flag float32 tensors keep the full-fp32 kernels: the results differ from the rounded ones
    exact = ops.gated_delta_scan(q, k, v, beta, g, 64, **kw)
    assert not torch.equal(exact, out)
    assert_close(exact, ref_out, TOL_F32, "out (fp32 kernels)")


def test_ir_op_records_take_flags_from_the_environment():
    """An unchanged op-60 record with float32 tensors reaches the tensor-core kernels when the process sets
    MXB_IR_GDN_FLAGS=64 (the variable is read once per process, hence the child process)."""
    import subprocess
    import sys
    code = r'''
import torch
from mixlab_b200 import ops
from oracle import inputs
B, T, H, K, V = 2, 200, 2, 128, 128
a = inputs.gdn_inputs(B, T, H, K, V, seed=5, io_dtype=torch.float32)
q, k, v, beta = (a[n].cuda() for n in ("q", "k", "v", "beta"))
gate = torch.exp(a["g"]).cuda()
out = ops.ir_op_forward(60, [q, k, v, beta, gate], [B, T, H, K, V, 64], out_shape=(B * T * H, V))
ref = ops.gated_delta_scan(q.bfloat16(), k.bfloat16(), v.bfloat16(), beta, gate, 64).float().reshape(B * T * H, V)
exact = ops.gated_delta_scan(q, k, v, beta, gate, 64).reshape(B * T * H, V)
assert torch.equal(out, ref), "record did not take the tensor-core kernels"
assert not torch.equal(out, exact)
print("IR_FLAGS_OK")
'''
    env = dict(os.environ, MXB_IR_GDN_FLAGS="64")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert "IR_FLAGS_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_host_buffer_entry_point_head_groups_on_tensor_core_kernels(monkeypatch):
    """Two sequences of eight 128-wide bf16 heads: by default the call cuts every sequence into two head groups (rows of
    a group stay >= 1 KB) and must return what the device entry points return on the whole tensors."""
    import ctypes as C
    lib = mixlab_b200.lib()
    B, T, H, K, V = 2, 200, 8, 128, 128
    a = inputs.gdn_inputs(B, T, H, K, V, seed=8, io_dtype=torch.bfloat16, with_grad_out=True)
    dev = {n: _dev(a[n]) for n in ("q", "k", "v", "beta", "g", "d_out")}
    want_out = ops.gated_delta_scan(dev["q"], dev["k"], dev["v"], dev["beta"], dev["g"], 64, gate_is_log=True)
    want = ops.gated_delta_scan_backward(dev["q"], dev["k"], dev["v"], dev["beta"], dev["g"], dev["d_out"], 64, gate_is_log=True)
    host = {n: a[n].contiguous().pin_memory() for n in ("q", "k", "v", "beta", "g", "d_out")}
    res = {n: torch.empty_like(host[m]).pin_memory() for n, m in
           (("out", "v"), ("dq", "q"), ("dk", "k"), ("dv", "v"), ("dbeta", "beta"), ("dgate", "g"))}
    p = lambda t: C.c_void_p(t.data_ptr())
    for split in (None, "1", "4"):
        if split is not None:
            monkeypatch.setenv("MXB_HOST_HEAD_SPLIT", split)
        ctx = C.c_void_p()
        assert lib.mxb_host_ctx_create(0, 256 << 20, C.byref(ctx)) == 0
        try:
            d = mixlab_b200.GdnDesc(B, T, H, K, V, 64, mixlab_b200.MXB_BF16, 1, 0)
            st = lib.mxb_host_gdn(ctx, C.byref(d), p(host["q"]), p(host["k"]), p(host["v"]), p(host["beta"]), p(host["g"]),
                                  p(res["out"]), p(host["d_out"]), p(res["dq"]), p(res["dk"]), p(res["dv"]), p(res["dbeta"]),
                                  p(res["dgate"]))
            assert st == 0
        finally:
            lib.mxb_host_ctx_destroy(ctx)
        # a head group is computed by the same kernels on the same numbers: bit-identical to the whole-tensor call
        assert torch.equal(res["out"], want_out.cpu()), split
        for n in ("dq", "dk", "dv", "dbeta", "dgate"):
            assert torch.equal(res[n], want[n].cpu()), (split, n)
