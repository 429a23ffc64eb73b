"""The workspace-free forward entry point (mxb_gdn_fwd_static_scratch).

Some hosts of this library cannot hand over a workspace because they cannot allocate
device memory at all (the device belongs to another runtime's pool) or must not call an
allocator where they run.  This checks, through the C ABI, that the variant with the
built-in scratch array gives the same output as the regular entry point - on two calls in
a row, since the second call finds the first call's leftovers in the array - and that it
refuses problems that do not fit.  Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

import mixlab_b200
from mixlab_b200 import _lib
from oracle import gdn, inputs
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _run_pair(lib, B, T, H, K, V, seed, io, extra_flags=0, check_oracle=True):
    a = inputs.gdn_inputs(B, T, H, K, V, seed=seed, io_dtype=io, with_h0=True)
    d = {k: v.cuda().contiguous() for k, v in a.items()}
    desc = mixlab_b200.GdnDesc(B, T, H, K, V, 64, _lib.MXB_F32 if io == torch.float32 else _lib.MXB_BF16, 1,
                               _lib.MXB_GDN_FORCE_FP32_PATH)
    # regular entry point with a torch-allocated workspace
    nws = lib.mxb_gdn_fwd_workspace_bytes(C.byref(desc))
    ws = torch.empty(nws, dtype=torch.uint8, device="cuda")
    out_ref, st_ref = torch.empty_like(d["v"]), torch.empty(B, H, K, V, device="cuda")
    assert lib.mxb_gdn_fwd(C.byref(desc), _p(d["q"]), _p(d["k"]), _p(d["v"]), _p(d["beta"]), _p(d["g"]), _p(d["h0"]),
                           _p(out_ref), _p(st_ref), _p(ws), nws, None) == 0
    # workspace-free entry point
    out, st = torch.full_like(d["v"], float("nan")), torch.full((B, H, K, V), float("nan"), device="cuda")
    desc2 = mixlab_b200.GdnDesc(B, T, H, K, V, 64, desc.io_dtype, 1, _lib.MXB_GDN_FORCE_FP32_PATH | extra_flags)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    assert lib.mxb_gdn_fwd_static_scratch(C.byref(desc2), _p(d["q"]), _p(d["k"]), _p(d["v"]), _p(d["beta"]), _p(d["g"]),
                                          _p(d["h0"]), _p(out), _p(st), None) == 0
    torch.cuda.synchronize()
    free1 = torch.cuda.mem_get_info()[0]
    tol = 1e-4 if io == torch.float32 else 2e-2
    assert_close(out, out_ref.double(), tol, "out vs mxb_gdn_fwd")
    assert_close(st, st_ref.double(), 1e-4, "state vs mxb_gdn_fwd")
    if not check_oracle:
        return free0, free1
    f = {k: v.double() for k, v in a.items()}
    want_o, want_s = gdn.scan_chunked(f["q"], f["k"], f["v"], f["beta"], torch.exp(f["g"]), 64, f["h0"])
    assert_close(out, want_o, tol, "out vs oracle")
    assert_close(st, want_s, tol, "state vs oracle")
    return free0, free1


def test_static_scratch_matches_regular_entry_point_twice():
    lib = mixlab_b200.lib()
    assert lib.mxb_gdn_static_scratch_bytes() == 16 << 20
    # two different problems back to back: the second reuses the array the first one dirtied
    _run_pair(lib, 2, 256, 4, 64, 64, seed=0, io=torch.float32)
    _run_pair(lib, 1, 130, 2, 128, 128, seed=1, io=torch.bfloat16)
    free0, free1 = _run_pair(lib, 2, 256, 4, 64, 64, seed=0, io=torch.float32)
    # by now the array's address is cached and the library's device code is loaded: the call itself must not
    # have taken any device memory (free memory as the driver reports it is the same before and after)
    assert free1 == free0, (free0, free1)


def test_static_scratch_ignores_save_for_backward():
    """A descriptor reused from a training forward may carry MXB_GDN_SAVE_FOR_BWD.  The saved tiles would not fit
    beside the forward scratch of this problem (about 14 MiB forward, 21 MiB with them): the flag must be ignored,
    not honoured past the end of the array."""
    lib = mixlab_b200.lib()
    B, T, H, K, V = 2, 1024, 7, 64, 64
    fwd_only = mixlab_b200.GdnDesc(B, T, H, K, V, 64, _lib.MXB_F32, 1, _lib.MXB_GDN_FORCE_FP32_PATH)
    with_save = mixlab_b200.GdnDesc(B, T, H, K, V, 64, _lib.MXB_F32, 1,
                                    _lib.MXB_GDN_FORCE_FP32_PATH | _lib.MXB_GDN_SAVE_FOR_BWD)
    assert lib.mxb_gdn_fwd_workspace_bytes(C.byref(fwd_only)) <= (16 << 20) < lib.mxb_gdn_fwd_workspace_bytes(C.byref(with_save))
    _run_pair(lib, B, T, H, K, V, seed=3, io=torch.float32, extra_flags=_lib.MXB_GDN_SAVE_FOR_BWD, check_oracle=False)


def test_static_scratch_rejects_oversized_problem():
    lib = mixlab_b200.lib()
    desc = mixlab_b200.GdnDesc(8, 4096, 16, 128, 128, 64, _lib.MXB_BF16, 1, 0)
    fake = C.c_void_p(4096)
    assert lib.mxb_gdn_fwd_static_scratch(C.byref(desc), fake, fake, fake, fake, fake, None, fake, None, None) == -3
    assert lib.mxb_gdn_fwd_static_scratch(None, fake, fake, fake, fake, fake, None, fake, None, None) == -1
