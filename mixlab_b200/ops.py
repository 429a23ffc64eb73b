"""Torch-tensor front end over the C ABI, named after the reference operators.

``gated_delta_scan`` mirrors ``Program.GatedDeltaScan`` (arch/ir.go:586-603):
inputs q,k [B,T,H,Dk], v [B,T,H,Dv], beta, gate [B,T,H], IntParams
[B,T,H,Dk,Dv,chunk]; ``mamba3_selective_scan`` mirrors
``Program.Mamba3SelectiveScan`` (arch/ir.go:528-553).  Every tensor must be a
contiguous CUDA tensor; nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import GdnDesc, Mamba3Desc, MXB_BF16, MXB_F32

_ws_cache: dict = {}
# (device index) -> token of the forward call whose saved intermediates the cached workspace holds; any other
# operator call on that device clears it, so that a backward with use_saved=True cannot consume overwritten tiles
_ws_saved: dict = {}


def _io(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return MXB_F32
    if t.dtype == torch.bfloat16:
        return MXB_BF16
    raise TypeError(f"unsupported dtype {t.dtype} (float32 or bfloat16)")


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("mixlab_b200 operators take CUDA tensors only (no CPU fallback)")
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    return C.c_void_p(t.data_ptr())


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("mixlab_b200 operators take CUDA tensors only (no CPU fallback)")


def _f32(t, name):
    if t is not None and t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32")
    return t


def _check_like(t, shape, dtype, device, name):
    """Raises unless ``t`` (None allowed) is a contiguous CUDA tensor of exactly this shape, dtype and device:
    the C ABI sees only pointers, so a wrong operand would otherwise be read out of bounds or as the wrong type."""
    if t is None:
        return
    if not t.is_cuda:
        raise ValueError("mixlab_b200 operators take CUDA tensors only (no CPU fallback)")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}")
    if t.dtype != dtype:
        raise TypeError(f"{name}: dtype {t.dtype}, expected {dtype}")
    if t.device != device:
        raise ValueError(f"{name}: on {t.device}, expected {device}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: tensor must be contiguous")


def _on_device_of_first(fn):
    """Runs ``fn`` with the device of its first tensor argument current: the stream handed to the C ABI and every
    allocation made inside then belong to the device the operands live on."""
    import functools

    @functools.wraps(fn)
    def wrapped(*args, **kw):
        first = args[0]
        if not torch.is_tensor(first) or not first.is_cuda:
            raise ValueError("mixlab_b200 operators take CUDA tensors only (no CPU fallback)")
        with torch.cuda.device(first.device):
            return fn(*args, **kw)
    return wrapped


def _check_all(device, *specs):
    for t, shape, dtype, name in specs:
        _check_like(t, shape, dtype, device, name)


def workspace(nbytes: int, device) -> torch.Tensor:
    """A cached byte buffer of at least ``nbytes`` on ``device`` (torch allocator)."""
    key = (device.index if device.index is not None else torch.cuda.current_device())
    _ws_saved.pop(key, None)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        _ws_cache.pop(key, None)
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev_key(device):
    return device.index if device.index is not None else torch.cuda.current_device()


def _saved_token(kind, tensors, extra):
    return (kind, torch.cuda.current_stream().cuda_stream, tuple((t.data_ptr(), tuple(t.shape), t.dtype) for t in tensors), extra)


def _mark_saved(device, token, ws):
    _ws_saved[_dev_key(device)] = (token, ws.data_ptr())


def _require_saved(device, token, what):
    """The (token, workspace address) pair of the forward whose intermediates a use_saved backward is about to
    consume; raises if any other operator call has used the cached workspace since."""
    rec = _ws_saved.get(_dev_key(device))
    if rec is None or rec[0] != token:
        raise RuntimeError(f"{what}: use_saved=True needs the immediately preceding save_for_backward forward on the "
                           "same tensors, stream and device (the cached workspace has been reused since, or never held them)")
    return rec


def _keep_saved(device, rec, ws, what):
    if ws.data_ptr() != rec[1]:
        raise RuntimeError(f"{what}: the cached workspace was reallocated after the forward saved into it")
    _ws_saved[_dev_key(device)] = rec


def _path_flags(flags):
    """The flag bits that choose a kernel family (and with it the layout of what a forward saves)."""
    return int(flags) & ~(_lib.MXB_GDN_SAVE_FOR_BWD | _lib.MXB_GDN_BWD_USE_SAVED)


def gdn_desc(q, v, chunk, gate_is_log, flags=0) -> GdnDesc:
    B, T, H, Dk = q.shape
    return GdnDesc(B, T, H, Dk, v.shape[-1], int(chunk), _io(q), int(bool(gate_is_log)), int(flags))


def _check_gdn(d, q, k, v, beta, gate, *, d_out=None, h0=None, d_final_state=None):
    if q.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k must be [B,T,H,Dk] and v [B,T,H,Dv]")
    dev, io, f32 = q.device, q.dtype, torch.float32
    _check_all(dev, (q, (d.B, d.T, d.H, d.Dk), io, "q"), (k, (d.B, d.T, d.H, d.Dk), io, "k"),
               (v, (d.B, d.T, d.H, d.Dv), io, "v"), (beta, (d.B, d.T, d.H), f32, "beta"),
               (gate, (d.B, d.T, d.H), f32, "gate"), (d_out, (d.B, d.T, d.H, d.Dv), io, "d_out"),
               (h0, (d.B, d.H, d.Dk, d.Dv), f32, "h0"), (d_final_state, (d.B, d.H, d.Dk, d.Dv), f32, "d_final_state"))


def gated_delta_scan(q, k, v, beta, gate, chunk=64, *, gate_is_log=False, h0=None,
                     return_final_state=False, flags=0, save_for_backward=False):
    """Forward.  Returns out [B,T,H,Dv] (and the final state [B,H,Dk,Dv] fp32).
    ``save_for_backward`` keeps the forward intermediates in the cached workspace for a
    following ``gated_delta_scan_backward(..., use_saved=True)`` on the same inputs."""
    if save_for_backward:
        flags |= _lib.MXB_GDN_SAVE_FOR_BWD
    _require_cuda(q, k, v, beta, gate, h0)
    l = _lib.lib()
    d = gdn_desc(q, v, chunk, gate_is_log, flags)
    _check_gdn(d, q, k, v, beta, gate, h0=h0)
    with torch.cuda.device(q.device):
        out = torch.empty_like(v)
        hT = torch.empty(d.B, d.H, d.Dk, d.Dv, dtype=torch.float32, device=q.device) if return_final_state else None
        nws = l.mxb_gdn_fwd_workspace_bytes(C.byref(d))
        ws = workspace(nws, q.device)
        _lib.check(l.mxb_gdn_fwd(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(gate), _ptr(h0), _ptr(out),
                                 _ptr(hT), _ptr(ws), ws.numel(), _stream()), "mxb_gdn_fwd")
        if save_for_backward:
            _mark_saved(q.device, _saved_token("gdn", (q, k, v, beta, gate), (int(chunk), bool(gate_is_log), _path_flags(flags))), ws)
    return (out, hT) if return_final_state else out


def gated_delta_scan_backward(q, k, v, beta, gate, d_out, chunk=64, *, gate_is_log=False, h0=None,
                              d_final_state=None, flags=0, use_saved=False):
    """All gradients.  Returns dict(dq, dk, dv, dbeta, dgate, dh0)."""
    if use_saved:
        flags |= _lib.MXB_GDN_BWD_USE_SAVED
    _require_cuda(q, k, v, beta, gate, d_out, h0, d_final_state)
    l = _lib.lib()
    d = gdn_desc(q, v, chunk, gate_is_log, flags)
    _check_gdn(d, q, k, v, beta, gate, d_out=d_out, h0=h0, d_final_state=d_final_state)
    with torch.cuda.device(q.device):
        saved = None
        if use_saved:
            saved = _require_saved(q.device, _saved_token("gdn", (q, k, v, beta, gate), (int(chunk), bool(gate_is_log), _path_flags(flags))),
                                   "gated_delta_scan_backward")
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dbeta, dgate = torch.empty_like(beta), torch.empty_like(gate)
        dh0 = torch.empty(d.B, d.H, d.Dk, d.Dv, dtype=torch.float32, device=q.device) if h0 is not None else None
        nws = l.mxb_gdn_bwd_workspace_bytes(C.byref(d))
        ws = workspace(nws, q.device)
        if saved is not None:
            _keep_saved(q.device, saved, ws, "gated_delta_scan_backward")
        _lib.check(l.mxb_gdn_bwd(C.byref(d), _ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(gate), _ptr(h0), _ptr(d_out),
                                 _ptr(d_final_state), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dbeta), _ptr(dgate), _ptr(dh0),
                                 _ptr(ws), ws.numel(), _stream()), "mxb_gdn_bwd")
    return dict(dq=dq, dk=dk, dv=dv, dbeta=dbeta, dgate=dgate, dh0=dh0)


def ir_op_forward(op_type: int, inputs, int_params, *, out_shape, float_params=()):
    """Runs one IR op record the way the reference's interpreter does after resolving its names
    (gpu/ir.cpp:4633-4654, :4837-4853): ``inputs`` in the record's order, IntParams as the Go side emits them
    (arch/ir.go:550-555, :600-602).  Returns the output tensor of ``out_shape`` in the dtype of the first input."""
    _require_cuda(*inputs)
    for i, t in enumerate(inputs):
        if not t.is_contiguous() or t.device != inputs[0].device:
            raise ValueError(f"input {i}: contiguous tensors on one device expected")
    l = _lib.lib()
    with torch.cuda.device(inputs[0].device):
        out = torch.empty(out_shape, dtype=inputs[0].dtype, device=inputs[0].device)
        ins = (C.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
        outs = (C.c_void_p * 1)(out.data_ptr())
        ip = (C.c_int32 * len(int_params))(*[int(v) for v in int_params])
        fp = (C.c_float * max(len(float_params), 1))(*[float(v) for v in float_params])
        rec = _lib.IrOp(int(op_type), ins, len(inputs), outs, 1, fp, len(float_params), ip, len(int_params), _io(inputs[0]))
        nws = l.mxb_ir_op_workspace_bytes(C.byref(rec))
        ws = workspace(nws, inputs[0].device)
        _lib.check(l.mxb_ir_op_forward(C.byref(rec), _ptr(ws), ws.numel(), _stream()), "mxb_ir_op_forward")
    return out


def device_status(device=None) -> int:
    """Blocking read of the device-side error word of the cached workspace (0 = ok)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    ws = workspace(256, dev)
    out = C.c_int32(0)
    _lib.check(_lib.lib().mxb_gdn_device_status(_ptr(ws), C.byref(out)), "mxb_gdn_device_status")
    return out.value


def gated_delta_decode_step(state, q, k, v, beta, gate, *, gate_is_log=False, out=None, flags=0):
    """One token on a persistent state [N,H,Dk,Dv] (updated in place).  Returns out [N,H,Dv]."""
    _require_cuda(state, q, k, v, beta, gate)
    l = _lib.lib()
    if state.dim() != 4:
        raise ValueError("state must be [N,H,Dk,Dv]")
    N, H, Dk, Dv = state.shape
    d = GdnDesc(N, 1, H, Dk, Dv, 0, _io(q), int(bool(gate_is_log)), int(flags))
    dev, io, f32 = state.device, q.dtype, torch.float32
    _check_all(dev, (state, (N, H, Dk, Dv), f32, "state"), (q, (N, H, Dk), io, "q"), (k, (N, H, Dk), io, "k"),
               (v, (N, H, Dv), io, "v"), (beta, (N, H), f32, "beta"), (gate, (N, H), f32, "gate"),
               (out, (N, H, Dv), io, "out"))
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty_like(v)
        _lib.check(l.mxb_gdn_decode_step(C.byref(d), _ptr(state), _ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(gate),
                                         _ptr(out), _stream()), "mxb_gdn_decode_step")
    return out


# ---------------------------------------------------------------- gated_deltanet block stages
def _block_desc(q_proj, H, Dk, Dv, gate_is_log):
    B, T, _ = q_proj.shape
    return GdnDesc(B, T, H, Dk, Dv, 64, _io(q_proj), int(bool(gate_is_log)), 0)


@_on_device_of_first
def gdn_block_pre(q_proj, k_proj, v_proj, conv_q, conv_k, conv_v, a_raw, b_raw, a_log, dt_bias, H, Dk, Dv, *,
                  gate_is_log=False):
    """Convolution + SiLU + L2-norm / gate / beta stage in front of the scan.  q_proj, k_proj [B,T,H*Dk],
    v_proj [B,T,H*Dv]; returns q, k [B,T,H,Dk], v [B,T,H,Dv] (I/O dtype), beta, gate [B,T,H] fp32."""
    _require_cuda(q_proj, k_proj, v_proj, conv_q, conv_k, conv_v, a_raw, b_raw, a_log, dt_bias)
    l = _lib.lib()
    d = _block_desc(q_proj, H, Dk, Dv, gate_is_log)
    dev, io, f = q_proj.device, q_proj.dtype, torch.float32
    _check_all(dev, (q_proj, (d.B, d.T, H * Dk), io, "q_proj"), (k_proj, (d.B, d.T, H * Dk), io, "k_proj"),
               (v_proj, (d.B, d.T, H * Dv), io, "v_proj"), (conv_q, (4, H * Dk), f, "conv_q"), (conv_k, (4, H * Dk), f, "conv_k"),
               (conv_v, (4, H * Dv), f, "conv_v"), (a_raw, (d.B, d.T, H), f, "a_raw"), (b_raw, (d.B, d.T, H), f, "b_raw"),
               (a_log, (H,), f, "a_log"), (dt_bias, (H,), f, "dt_bias"))
    B, T = d.B, d.T
    q = torch.empty(B, T, H, Dk, dtype=q_proj.dtype, device=q_proj.device)
    k = torch.empty_like(q)
    v = torch.empty(B, T, H, Dv, dtype=q_proj.dtype, device=q_proj.device)
    beta = torch.empty(B, T, H, dtype=torch.float32, device=q_proj.device)
    gate = torch.empty_like(beta)
    _lib.check(l.mxb_gdn_block_pre_fwd(C.byref(d), _ptr(q_proj), _ptr(k_proj), _ptr(v_proj), _ptr(_f32(conv_q, "conv_q")),
                                       _ptr(_f32(conv_k, "conv_k")), _ptr(_f32(conv_v, "conv_v")),
                                       _ptr(_f32(a_raw, "a_raw")), _ptr(_f32(b_raw, "b_raw")), _ptr(_f32(a_log, "a_log")),
                                       _ptr(_f32(dt_bias, "dt_bias")), _ptr(q), _ptr(k), _ptr(v), _ptr(beta), _ptr(gate),
                                       _stream()), "mxb_gdn_block_pre_fwd")
    return q, k, v, beta, gate


@_on_device_of_first
def gdn_block_pre_backward(q_proj, k_proj, v_proj, conv_q, conv_k, conv_v, a_raw, b_raw, a_log, dt_bias, H, Dk, Dv,
                           dq, dk, dv, dbeta, dgate, *, gate_is_log=False):
    """Gradients of gdn_block_pre: dict(dq_proj, dk_proj, dv_proj, dconv_q, dconv_k, dconv_v, da_raw, db_raw, da_log,
    ddt_bias)."""
    _require_cuda(q_proj, k_proj, v_proj, conv_q, conv_k, conv_v, a_raw, b_raw, a_log, dt_bias, dq, dk, dv, dbeta, dgate)
    l = _lib.lib()
    d = _block_desc(q_proj, H, Dk, Dv, gate_is_log)
    dev, io, f = q_proj.device, q_proj.dtype, torch.float32
    _check_all(dev, (q_proj, (d.B, d.T, H * Dk), io, "q_proj"), (k_proj, (d.B, d.T, H * Dk), io, "k_proj"),
               (v_proj, (d.B, d.T, H * Dv), io, "v_proj"), (conv_q, (4, H * Dk), f, "conv_q"), (conv_k, (4, H * Dk), f, "conv_k"),
               (conv_v, (4, H * Dv), f, "conv_v"), (a_raw, (d.B, d.T, H), f, "a_raw"), (b_raw, (d.B, d.T, H), f, "b_raw"),
               (a_log, (H,), f, "a_log"), (dt_bias, (H,), f, "dt_bias"), (dq, (d.B, d.T, H, Dk), io, "dq"),
               (dk, (d.B, d.T, H, Dk), io, "dk"), (dv, (d.B, d.T, H, Dv), io, "dv"), (dbeta, (d.B, d.T, H), f, "dbeta"),
               (dgate, (d.B, d.T, H), f, "dgate"))
    dqp, dkp, dvp = torch.empty_like(q_proj), torch.empty_like(k_proj), torch.empty_like(v_proj)
    f32 = dict(dtype=torch.float32, device=q_proj.device)
    dcq, dck, dcv = torch.empty(4, H * Dk, **f32), torch.empty(4, H * Dk, **f32), torch.empty(4, H * Dv, **f32)
    da, db = torch.empty(d.B, d.T, H, **f32), torch.empty(d.B, d.T, H, **f32)
    dal, dbias = torch.empty(H, **f32), torch.empty(H, **f32)
    ws = workspace(l.mxb_gdn_block_workspace_bytes(C.byref(d)), q_proj.device)
    _lib.check(l.mxb_gdn_block_pre_bwd(C.byref(d), _ptr(q_proj), _ptr(k_proj), _ptr(v_proj), _ptr(_f32(conv_q, "conv_q")),
                                       _ptr(_f32(conv_k, "conv_k")), _ptr(_f32(conv_v, "conv_v")),
                                       _ptr(_f32(a_raw, "a_raw")), _ptr(_f32(b_raw, "b_raw")), _ptr(_f32(a_log, "a_log")),
                                       _ptr(_f32(dt_bias, "dt_bias")), _ptr(dq), _ptr(dk), _ptr(dv),
                                       _ptr(_f32(dbeta, "dbeta")), _ptr(_f32(dgate, "dgate")), _ptr(dqp), _ptr(dkp),
                                       _ptr(dvp), _ptr(dcq), _ptr(dck), _ptr(dcv), _ptr(da), _ptr(db), _ptr(dal),
                                       _ptr(dbias), _ptr(ws), ws.numel(), _stream()), "mxb_gdn_block_pre_bwd")
    return dict(dq_proj=dqp, dk_proj=dkp, dv_proj=dvp, dconv_q=dcq, dconv_k=dck, dconv_v=dcv, da_raw=da, db_raw=db,
                da_log=dal, ddt_bias=dbias)


@_on_device_of_first
def gdn_block_post(o, z, o_norm):
    """y = RMSNorm(o, o_norm, 1e-5) * SiLU(z).  o [B,T,H,Dv], z [B,T,H*Dv] -> y [B,T,H*Dv]."""
    _require_cuda(o, z, o_norm)
    l = _lib.lib()
    B, T, H, Dv = o.shape
    d = GdnDesc(B, T, H, 8, Dv, 64, _io(o), 0, 0)
    _check_all(o.device, (o, (B, T, H, Dv), o.dtype, "o"), (z, (B, T, H * Dv), o.dtype, "z"),
               (o_norm, (Dv,), torch.float32, "o_norm"))
    y = torch.empty_like(z)
    _lib.check(l.mxb_gdn_block_post_fwd(C.byref(d), _ptr(o), _ptr(z), _ptr(_f32(o_norm, "o_norm")), _ptr(y), _stream()),
               "mxb_gdn_block_post_fwd")
    return y


@_on_device_of_first
def gdn_block_post_backward(o, z, o_norm, dy):
    """Gradients of gdn_block_post: dict(do, dz, do_norm)."""
    _require_cuda(o, z, o_norm, dy)
    l = _lib.lib()
    B, T, H, Dv = o.shape
    d = GdnDesc(B, T, H, 8, Dv, 64, _io(o), 0, 0)
    _check_all(o.device, (o, (B, T, H, Dv), o.dtype, "o"), (z, (B, T, H * Dv), o.dtype, "z"),
               (o_norm, (Dv,), torch.float32, "o_norm"), (dy, (B, T, H * Dv), o.dtype, "dy"))
    d_o, dz = torch.empty_like(o), torch.empty_like(z)
    dw = torch.empty(Dv, dtype=torch.float32, device=o.device)
    ws = workspace(l.mxb_gdn_block_workspace_bytes(C.byref(d)), o.device)
    _lib.check(l.mxb_gdn_block_post_bwd(C.byref(d), _ptr(o), _ptr(z), _ptr(_f32(o_norm, "o_norm")), _ptr(dy), _ptr(d_o),
                                        _ptr(dz), _ptr(dw), _ptr(ws), ws.numel(), _stream()), "mxb_gdn_block_post_bwd")
    return dict(do=d_o, dz=dz, do_norm=dw)


def _check_mamba3(d, x, dt, lam, theta, a_log, b, c, dy=None):
    dev, io, f = x.device, x.dtype, torch.float32
    if d.nheads > 0:
        per, th, al = (d.B, d.T, d.nheads), (d.B, d.T, d.nheads), (d.nheads,)
    else:
        per, th, al = (d.B, d.T, d.D), (d.B, d.T, d.D, d.N // 2), (d.D, d.N)
    _check_all(dev, (x, (d.B, d.T, d.D), io, "x"), (dt, per, f, "dt"), (lam, per, f, "lambda"), (theta, th, f, "theta"),
               (a_log, al, f, "a_log"), (b, (d.B, d.T, d.G, d.N), io, "b"), (c, (d.B, d.T, d.G, d.N), io, "c"),
               (dy, (d.B, d.T, d.D), io, "dy"))


def mamba3_desc(x, b, nheads, flags=0) -> Mamba3Desc:
    if x.dim() != 3 or b.dim() != 4:
        raise ValueError("x must be [B,T,D] and b, c [B,T,G,N]")
    B, T, D = x.shape
    G, N = b.shape[-2], b.shape[-1]
    return Mamba3Desc(B, T, D, N, G, int(nheads), _io(x), int(flags))


@_on_device_of_first
def mamba3_selective_scan(x, dt, lam, theta, a_log, b, c, *, nheads=0, flags=0, save_for_backward=False):
    """Forward.  x [B,T,D]; b,c [B,T,G,N]; per-channel (nheads=0) or head-broadcast parameters.
    ``save_for_backward`` keeps the chunk states in the cached workspace for a following
    ``mamba3_selective_scan_backward(..., use_saved=True)`` on the same inputs."""
    if save_for_backward:
        flags |= _lib.MXB_MAMBA3_SAVE_FOR_BWD
    _require_cuda(x, dt, lam, theta, a_log, b, c)
    l = _lib.lib()
    d = mamba3_desc(x, b, nheads, flags)
    _check_mamba3(d, x, dt, lam, theta, a_log, b, c)
    y = torch.empty_like(x)
    nws = l.mxb_mamba3_fwd_workspace_bytes(C.byref(d))
    ws = workspace(nws, x.device)
    _lib.check(l.mxb_mamba3_fwd(C.byref(d), _ptr(x), _ptr(_f32(dt, "dt")), _ptr(_f32(lam, "lambda")),
                                _ptr(_f32(theta, "theta")), _ptr(_f32(a_log, "a_log")), _ptr(b), _ptr(c),
                                _ptr(y), _ptr(ws), ws.numel(), _stream()), "mxb_mamba3_fwd")
    if save_for_backward:
        _mark_saved(x.device, _saved_token("mamba3", (x, dt, lam, theta, a_log, b, c), int(nheads)), ws)
    return y


@_on_device_of_first
def mamba3_selective_scan_backward(x, dt, lam, theta, a_log, b, c, dy, *, nheads=0, flags=0, use_saved=False):
    """Gradients in argument order.  Returns dict(dx, ddt, dlambda, dtheta, da_log, db, dc)."""
    if use_saved:
        flags |= _lib.MXB_MAMBA3_BWD_USE_SAVED
    _require_cuda(x, dt, lam, theta, a_log, b, c, dy)
    l = _lib.lib()
    d = mamba3_desc(x, b, nheads, flags)
    _check_mamba3(d, x, dt, lam, theta, a_log, b, c, dy)
    saved = None
    if use_saved:
        saved = _require_saved(x.device, _saved_token("mamba3", (x, dt, lam, theta, a_log, b, c), int(nheads)),
                               "mamba3_selective_scan_backward")
    dx = torch.empty_like(x)
    ddt, dlam, dth, dal = (torch.empty_like(t) for t in (dt, lam, theta, a_log))
    db, dc = torch.empty_like(b), torch.empty_like(c)
    nws = l.mxb_mamba3_bwd_workspace_bytes(C.byref(d))
    ws = workspace(nws, x.device)
    if saved is not None:
        _keep_saved(x.device, saved, ws, "mamba3_selective_scan_backward")
    _lib.check(l.mxb_mamba3_bwd(C.byref(d), _ptr(x), _ptr(_f32(dt, "dt")), _ptr(_f32(lam, "lambda")),
                                _ptr(_f32(theta, "theta")), _ptr(_f32(a_log, "a_log")), _ptr(b), _ptr(c),
                                _ptr(dy), _ptr(dx), _ptr(ddt), _ptr(dlam), _ptr(dth), _ptr(dal), _ptr(db),
                                _ptr(dc), _ptr(ws), ws.numel(), _stream()), "mxb_mamba3_bwd")
    return dict(dx=dx, ddt=ddt, dlambda=dlam, dtheta=dth, da_log=dal, db=db, dc=dc)


# ---------------------------------------------------------------- Mamba-3 block stages
def _m3_block_desc(x, N, G):
    B, T, D = x.shape
    return Mamba3Desc(B, T, D, int(N), int(G), 0, _io(x), 0)


@_on_device_of_first
def mamba3_block_conv(x, w):
    """Causal depthwise convolution: x [B,T,D], w [D,K] (K <= 4; tap k multiplies x[t-k])."""
    _require_cuda(x, w)
    l = _lib.lib()
    d = _m3_block_desc(x, 8, 1)
    _check_all(x.device, (x, (d.B, d.T, d.D), x.dtype, "x"), (w, (d.D, w.shape[-1]), torch.float32, "w"))
    y = torch.empty_like(x)
    _lib.check(l.mxb_mamba3_block_conv_fwd(C.byref(d), int(w.shape[1]), _ptr(x), _ptr(_f32(w, "w")), _ptr(y), _stream()),
               "mxb_mamba3_block_conv_fwd")
    return y


@_on_device_of_first
def mamba3_block_conv_backward(x, w, dy):
    _require_cuda(x, w, dy)
    l = _lib.lib()
    d = _m3_block_desc(x, 8, 1)
    _check_all(x.device, (x, (d.B, d.T, d.D), x.dtype, "x"), (w, (d.D, w.shape[-1]), torch.float32, "w"),
               (dy, (d.B, d.T, d.D), x.dtype, "dy"))
    dx = torch.empty_like(x)
    dw = torch.empty(w.shape, dtype=torch.float32, device=x.device)
    ws = workspace(l.mxb_mamba3_block_workspace_bytes(C.byref(d)), x.device)
    _lib.check(l.mxb_mamba3_block_conv_bwd(C.byref(d), int(w.shape[1]), _ptr(x), _ptr(_f32(w, "w")), _ptr(dy), _ptr(dx),
                                           _ptr(dw), _ptr(ws), ws.numel(), _stream()), "mxb_mamba3_block_conv_bwd")
    return dict(dx=dx, dw=dw)


@_on_device_of_first
def mamba3_block_bc(b_proj, c_proj, b_scale, c_scale, b_bias, c_bias, G, N, eps=1e-5):
    """b = RMSNorm(b_proj rows of N, b_scale, eps) + b_bias, same for c.  [B,T,G*N] -> [B,T,G,N]."""
    _require_cuda(b_proj, c_proj, b_scale, c_scale, b_bias, c_bias)
    l = _lib.lib()
    B, T, _ = b_proj.shape
    d = Mamba3Desc(B, T, 8, int(N), int(G), 0, _io(b_proj), 0)
    dev, io, f = b_proj.device, b_proj.dtype, torch.float32
    _check_all(dev, (b_proj, (B, T, G * N), io, "b_proj"), (c_proj, (B, T, G * N), io, "c_proj"), (b_scale, (N,), f, "b_scale"),
               (c_scale, (N,), f, "c_scale"), (b_bias, (G * N,), f, "b_bias"), (c_bias, (G * N,), f, "c_bias"))
    b = torch.empty(B, T, G, N, dtype=b_proj.dtype, device=b_proj.device)
    c = torch.empty_like(b)
    _lib.check(l.mxb_mamba3_block_bc_fwd(C.byref(d), float(eps), _ptr(b_proj), _ptr(c_proj), _ptr(_f32(b_scale, "b_scale")),
                                         _ptr(_f32(c_scale, "c_scale")), _ptr(_f32(b_bias, "b_bias")),
                                         _ptr(_f32(c_bias, "c_bias")), _ptr(b), _ptr(c), _stream()), "mxb_mamba3_block_bc_fwd")
    return b, c


@_on_device_of_first
def mamba3_block_bc_backward(b_proj, c_proj, b_scale, c_scale, db, dc, G, N, eps=1e-5):
    _require_cuda(b_proj, c_proj, b_scale, c_scale, db, dc)
    l = _lib.lib()
    B, T, _ = b_proj.shape
    d = Mamba3Desc(B, T, 8, int(N), int(G), 0, _io(b_proj), 0)
    dev, io, f = b_proj.device, b_proj.dtype, torch.float32
    _check_all(dev, (b_proj, (B, T, G * N), io, "b_proj"), (c_proj, (B, T, G * N), io, "c_proj"), (b_scale, (N,), f, "b_scale"),
               (c_scale, (N,), f, "c_scale"), (db, (B, T, G, N), io, "db"), (dc, (B, T, G, N), io, "dc"))
    dbp, dcp = torch.empty_like(b_proj), torch.empty_like(c_proj)
    f32 = dict(dtype=torch.float32, device=b_proj.device)
    dbs, dcs, dbb, dcb = torch.empty(N, **f32), torch.empty(N, **f32), torch.empty(G * N, **f32), torch.empty(G * N, **f32)
    ws = workspace(l.mxb_mamba3_block_workspace_bytes(C.byref(d)), b_proj.device)
    _lib.check(l.mxb_mamba3_block_bc_bwd(C.byref(d), float(eps), _ptr(b_proj), _ptr(c_proj), _ptr(_f32(b_scale, "b_scale")),
                                         _ptr(_f32(c_scale, "c_scale")), _ptr(db), _ptr(dc), _ptr(dbp), _ptr(dcp), _ptr(dbs),
                                         _ptr(dcs), _ptr(dbb), _ptr(dcb), _ptr(ws), ws.numel(), _stream()),
               "mxb_mamba3_block_bc_bwd")
    return dict(db_proj=dbp, dc_proj=dcp, db_scale=dbs, dc_scale=dcs, db_bias=dbb, dc_bias=dcb)


@_on_device_of_first
def mamba3_block_post(y, z, post_norm, eps=1e-5):
    """RMSNorm(y rows of D, post_norm, eps) * z * sigmoid(z).  y, z [B,T,D]."""
    _require_cuda(y, z, post_norm)
    l = _lib.lib()
    d = _m3_block_desc(y, 8, 1)
    _check_all(y.device, (y, (d.B, d.T, d.D), y.dtype, "y"), (z, (d.B, d.T, d.D), y.dtype, "z"),
               (post_norm, (d.D,), torch.float32, "post_norm"))
    out = torch.empty_like(y)
    _lib.check(l.mxb_mamba3_block_post_fwd(C.byref(d), float(eps), _ptr(y), _ptr(z), _ptr(_f32(post_norm, "post_norm")),
                                           _ptr(out), _stream()), "mxb_mamba3_block_post_fwd")
    return out


@_on_device_of_first
def mamba3_block_post_backward(y, z, post_norm, dout, eps=1e-5):
    _require_cuda(y, z, post_norm, dout)
    l = _lib.lib()
    d = _m3_block_desc(y, 8, 1)
    _check_all(y.device, (y, (d.B, d.T, d.D), y.dtype, "y"), (z, (d.B, d.T, d.D), y.dtype, "z"),
               (post_norm, (d.D,), torch.float32, "post_norm"), (dout, (d.B, d.T, d.D), y.dtype, "dout"))
    dy, dz = torch.empty_like(y), torch.empty_like(z)
    dw = torch.empty(y.shape[-1], dtype=torch.float32, device=y.device)
    ws = workspace(l.mxb_mamba3_block_workspace_bytes(C.byref(d)), y.device)
    _lib.check(l.mxb_mamba3_block_post_bwd(C.byref(d), float(eps), _ptr(y), _ptr(z), _ptr(_f32(post_norm, "post_norm")),
                                           _ptr(dout), _ptr(dy), _ptr(dz), _ptr(dw), _ptr(ws), ws.numel(), _stream()),
               "mxb_mamba3_block_post_bwd")
    return dict(dy=dy, dz=dz, dpost_norm=dw)
