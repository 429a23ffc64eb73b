"""C-ABI checks that need no GPU: the library loads, exports exactly what the
header declares, and rejects bad arguments before touching a device."""
import ctypes as C
import os
import re

import pytest

import mixlab_b200
from mixlab_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    text = open(os.path.join(ROOT, "include", "mixlab_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"MXB_API\s+[\w\s\*]+?\b(mxb_\w+)\s*\(", text))


def test_library_exports_match_header():
    lib = mixlab_b200.load_library()
    declared = _header_functions()
    assert declared, "no MXB_API declarations found"
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_version_and_status_strings():
    lib = mixlab_b200.lib()
    assert lib.mxb_version() >= 100
    for s in (0, -1, -2, -3, -4, -5, -6):
        assert lib.mxb_status_string(s)
    assert b"unknown" in lib.mxb_status_string(-99)


def test_gdn_argument_errors():
    lib = mixlab_b200.lib()
    d = mixlab_b200.GdnDesc(2, 16, 2, 8, 8, 64, _lib.MXB_F32, 0, 0)
    assert lib.mxb_gdn_fwd(None, *([None] * 9), 0, None) == -1
    assert lib.mxb_gdn_fwd(C.byref(d), *([None] * 9), 0, None) == -1           # null tensors
    bad = mixlab_b200.GdnDesc(2, 16, 2, 8, 8, 64, 7, 0, 0)                    # bad dtype
    assert lib.mxb_gdn_fwd_workspace_bytes(C.byref(bad)) == 0
    fake = C.c_void_p(4096)
    assert lib.mxb_gdn_fwd(C.byref(bad), fake, fake, fake, fake, fake, None, fake, None, None, 0, None) == -1
    # workspace too small is reported before any launch
    assert lib.mxb_gdn_fwd_workspace_bytes(C.byref(d)) > 0
    assert lib.mxb_gdn_fwd(C.byref(d), fake, fake, fake, fake, fake, None, fake, None, None, 0, None) == -3
    assert lib.mxb_gdn_bwd(C.byref(d), *([fake] * 6), fake, None, *([fake] * 5), None, None, 0, None) == -3
    big = mixlab_b200.GdnDesc(1, 16, 1, 512, 512, 64, _lib.MXB_F32, 0, 0)     # beyond every kernel
    n = lib.mxb_gdn_fwd_workspace_bytes(C.byref(big))
    assert lib.mxb_gdn_fwd(C.byref(big), fake, fake, fake, fake, fake, None, fake, None, fake, n, None) == -2


def test_workspace_sizes_scale():
    lib = mixlab_b200.lib()
    a = mixlab_b200.GdnDesc(1, 256, 4, 64, 64, 64, _lib.MXB_F32, 0, 0)
    b = mixlab_b200.GdnDesc(2, 256, 4, 64, 64, 64, _lib.MXB_F32, 0, 0)
    fa, fb = lib.mxb_gdn_fwd_workspace_bytes(C.byref(a)), lib.mxb_gdn_fwd_workspace_bytes(C.byref(b))
    assert 0 < fa < fb <= 2 * fa + 4096
    assert lib.mxb_gdn_bwd_workspace_bytes(C.byref(a)) > fa
    naive = mixlab_b200.GdnDesc(1, 256, 4, 64, 64, 0, _lib.MXB_F32, 0, 0)
    assert lib.mxb_gdn_fwd_workspace_bytes(C.byref(naive)) == 0


def test_mamba3_argument_errors():
    lib = mixlab_b200.lib()
    fake = C.c_void_p(4096)
    odd = mixlab_b200.Mamba3Desc(1, 8, 4, 7, 1, 0, _lib.MXB_F32, 0)          # odd state size
    assert lib.mxb_mamba3_fwd(C.byref(odd), *([fake] * 8), None, 0, None) == -2
    ok = mixlab_b200.Mamba3Desc(1, 8, 4, 8, 2, 0, _lib.MXB_F32, 0)
    assert lib.mxb_mamba3_fwd(C.byref(ok), *([None] * 8), None, 0, None) == -1
    assert lib.mxb_mamba3_bwd_workspace_bytes(C.byref(ok)) > 0
    assert lib.mxb_mamba3_bwd(C.byref(ok), *([fake] * 15), None, 0, None) == -3
    grp = mixlab_b200.Mamba3Desc(1, 8, 6, 8, 4, 0, _lib.MXB_F32, 0)          # D % G != 0
    assert lib.mxb_mamba3_fwd(C.byref(grp), *([fake] * 8), None, 0, None) == -2


def test_ops_refuse_cpu_tensors():
    import torch
    q = torch.zeros(1, 4, 1, 8)
    with pytest.raises(ValueError):
        mixlab_b200.ops.gated_delta_scan(q, q, q, torch.zeros(1, 4, 1), torch.ones(1, 4, 1), 64)


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(ImportError):
        mixlab_b200.load_library(str(tmp_path / "nope.so"))
