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


def test_tensor_core_paths_reject_unaligned_pointers():
    """The tensor-core kernels move whole 16-byte units: a q/k/v/out (x/b/c/y) base that is not 16-byte aligned is
    refused at the C ABI, before any launch (fake pointers: nothing is dereferenced)."""
    lib = mixlab_b200.lib()
    ok, odd = C.c_void_p(1 << 20), C.c_void_p((1 << 20) + 8)
    d = mixlab_b200.GdnDesc(1, 128, 2, 128, 128, 64, _lib.MXB_BF16, 1, 0)        # tensor-core shape
    n = lib.mxb_gdn_bwd_workspace_bytes(C.byref(d))
    for bad in range(3):
        a = [ok, ok, ok]
        a[bad] = odd
        assert lib.mxb_gdn_fwd(C.byref(d), *a, ok, ok, None, ok, None, ok, n, None) == -5
        assert lib.mxb_gdn_bwd(C.byref(d), *a, ok, ok, None, ok, None, ok, ok, ok, ok, ok, None, ok, n, None) == -5
    assert lib.mxb_gdn_fwd(C.byref(d), ok, ok, ok, ok, ok, None, odd, None, ok, n, None) == -5
    assert lib.mxb_gdn_bwd(C.byref(d), ok, ok, ok, ok, ok, None, odd, None, ok, ok, ok, ok, ok, None, ok, n, None) == -5
    assert lib.mxb_gdn_bwd(C.byref(d), ok, ok, ok, ok, ok, None, ok, None, ok, odd, ok, ok, ok, None, ok, n, None) == -5
    m = mixlab_b200.Mamba3Desc(1, 128, 128, 128, 1, 2, _lib.MXB_BF16, 0)         # chunked tensor-core shape
    nm = lib.mxb_mamba3_bwd_workspace_bytes(C.byref(m))
    assert nm > 0
    assert lib.mxb_mamba3_fwd(C.byref(m), odd, ok, ok, ok, ok, ok, ok, ok, ok, nm, None) == -5
    assert lib.mxb_mamba3_fwd(C.byref(m), ok, ok, ok, ok, ok, odd, ok, ok, ok, nm, None) == -5
    assert lib.mxb_mamba3_bwd(C.byref(m), ok, ok, ok, ok, ok, ok, ok, odd, *([ok] * 7), ok, nm, None) == -5


def test_chunk_above_64_is_accepted():
    lib = mixlab_b200.lib()
    d64 = mixlab_b200.GdnDesc(1, 256, 2, 32, 32, 64, _lib.MXB_F32, 0, 0)
    d128 = mixlab_b200.GdnDesc(1, 256, 2, 32, 32, 128, _lib.MXB_F32, 0, 0)
    assert lib.mxb_gdn_fwd_workspace_bytes(C.byref(d128)) == lib.mxb_gdn_fwd_workspace_bytes(C.byref(d64)) > 0
    wide = mixlab_b200.GdnDesc(1, 64, 1, 128, 256, 64, _lib.MXB_F32, 0, 0)     # the reference default Dv = 2 Dk
    assert lib.mxb_gdn_bwd_workspace_bytes(C.byref(wide)) > 0


def test_ops_check_every_operand():
    """Shape, dtype and device of every operand are checked in Python before the C ABI sees a pointer.  The checks
    run before the CUDA requirement is looked at only for CUDA tensors, so this uses the helper directly."""
    import torch
    from mixlab_b200 import ops
    dev = torch.device("cpu")
    t = torch.zeros(2, 3)

    class FakeCuda:
        """Stands in for a CUDA tensor: only the attributes the checker reads."""
        def __init__(self, shape, dtype, device="cuda:0", contiguous=True):
            self.shape, self.dtype, self.device, self._c, self.is_cuda = shape, dtype, device, contiguous, True

        def is_contiguous(self):
            return self._c

    good = FakeCuda((2, 3), torch.float32)
    ops._check_like(good, (2, 3), torch.float32, "cuda:0", "x")
    ops._check_like(None, (2, 3), torch.float32, "cuda:0", "x")
    with pytest.raises(ValueError):
        ops._check_like(t, (2, 3), torch.float32, dev, "x")                              # not a CUDA tensor
    with pytest.raises(ValueError):
        ops._check_like(FakeCuda((2, 4), torch.float32), (2, 3), torch.float32, "cuda:0", "x")
    with pytest.raises(TypeError):
        ops._check_like(FakeCuda((2, 3), torch.bfloat16), (2, 3), torch.float32, "cuda:0", "x")
    with pytest.raises(ValueError):
        ops._check_like(FakeCuda((2, 3), torch.float32, "cuda:1"), (2, 3), torch.float32, "cuda:0", "x")
    with pytest.raises(ValueError):
        ops._check_like(FakeCuda((2, 3), torch.float32, contiguous=False), (2, 3), torch.float32, "cuda:0", "x")


def test_ir_op_records_are_validated_like_the_interpreter():
    """mxb_ir_op mirrors mlx_ir_program_add_op records (gpu/mlx_bridge.h:83-89); the argument rules are the
    interpreter's (gpu/ir.cpp:4633-4654, :4837-4853).  Fake pointers: every case returns before a launch."""
    lib = mixlab_b200.lib()
    fake = 1 << 20

    def rec(op_type, n_in, ints, n_out=1):
        ins = (C.c_void_p * max(n_in, 1))(*([fake] * max(n_in, 1)))
        outs = (C.c_void_p * 1)(fake)
        ip = (C.c_int32 * max(len(ints), 1))(*ints) if ints else (C.c_int32 * 1)(0)
        r = _lib.IrOp(op_type, ins, n_in, outs, n_out, None, 0, ip, len(ints), _lib.MXB_F32)
        r._keep = (ins, outs, ip)
        return r

    ok60 = rec(60, 5, [2, 16, 2, 8, 8, 64])
    assert lib.mxb_ir_op_workspace_bytes(C.byref(ok60)) > 0
    assert lib.mxb_ir_op_forward(C.byref(ok60), None, 0, None) == -3                 # valid record, no workspace given
    assert lib.mxb_ir_op_workspace_bytes(C.byref(rec(60, 5, [2, 16, 2, 8, 8]))) == 0  # no chunk = recurrence: no workspace
    assert lib.mxb_ir_op_forward(C.byref(rec(60, 5, [2, 16, 2, 8])), None, 0, None) == -1     # "requires B,T,H,Dk,Dv"
    assert lib.mxb_ir_op_forward(C.byref(rec(60, 4, [2, 16, 2, 8, 8, 64])), None, 0, None) == -1
    assert lib.mxb_ir_op_forward(C.byref(rec(60, 5, [2, 16, 2, 8, 8, 64], n_out=0)), None, 0, None) == -1
    ok63 = rec(63, 7, [1, 8, 4, 8, 2])
    assert lib.mxb_ir_op_workspace_bytes(C.byref(ok63)) == 0 or lib.mxb_ir_op_workspace_bytes(C.byref(ok63)) > 0
    assert lib.mxb_ir_op_forward(C.byref(rec(63, 6, [1, 8, 4, 8, 2])), None, 0, None) == -1   # "requires 7 inputs"
    assert lib.mxb_ir_op_forward(C.byref(rec(63, 7, [1, 8, 4, 8])), None, 0, None) == -1
    assert lib.mxb_ir_op_forward(C.byref(rec(61, 5, [2, 16, 2, 8, 8])), None, 0, None) == -2   # another op of the IR
    assert lib.mxb_ir_op_forward(None, None, 0, None) == -1
