"""The fused element-wise passes of the data-parallel gradient exchange (mxb_dp_*) against plain torch ops, and one
staged step on a one-rank NCCL group against the reference's formulae (gpu/distributed_step.cpp:120-249,
gpu/optimizer_step_guard.cpp:76-104)."""
import ctypes as C
import math
import os
import socket

import pytest
import torch

import mixlab_b200

pytestmark = pytest.mark.gpu


def _p(t, off=0):
    return C.c_void_p(t.data_ptr() + 4 * off)


@pytest.mark.parametrize("n,offset", [(1, 0), (7, 1), (4099, 3), (1 << 20, 0), (3 * (1 << 20) + 5, 2)])
def test_dp_passes_match_torch(n, offset):
    lib = mixlab_b200.lib()
    g = torch.Generator(device="cuda").manual_seed(n)
    base = torch.randn(n + offset + 8, device="cuda", generator=g)
    x = base[offset:offset + n]           # deliberately not 16-byte aligned for offset != 0
    if n > 6:
        x[3] = float("nan"); x[n - 2] = float("inf"); x[n // 2] = float("-inf")
    ref = x.clone()
    aux = torch.zeros(4 + lib.mxb_dp_partial_floats(), device="cuda")
    assert lib.mxb_dp_sanitize(_p(x), n, 0.5, _p(aux), None) == 0
    fin = torch.isfinite(ref)
    want = torch.where(fin, ref * 0.5, torch.zeros_like(ref))
    assert torch.equal(x, want) and aux[0].item() == (0.0 if fin.all() else 1.0)
    assert torch.equal(base[offset + n:], base[offset + n:]) and torch.isfinite(base[offset + n:]).all()  # nothing past the end
    # finalize: divide, count, sum of squares, clip scale; then the scale pass
    if n > 6:
        x[5] = float("inf")
    y = x.clone()
    assert lib.mxb_dp_finalize(_p(x), n, 1.0 / 3.0, 2.0, _p(aux, 4), _p(aux, 1), None) == 0
    yd = y * (1.0 / 3.0)
    finy = torch.isfinite(yd)
    wanty = torch.where(finy, yd, torch.zeros_like(yd))
    assert torch.equal(x, wanty)
    assert aux[2].item() == float((~finy).sum())
    assert abs(aux[1].item() - wanty.double().pow(2).sum().item()) <= 1e-4 * max(1.0, wanty.double().pow(2).sum().item())
    assert aux[3].item() == (0.0 if (~finy).any() else min(1.0, 2.0 / (math.sqrt(aux[1].item()) + 1e-6)))
    # same inputs (at the same alignment), same bits: the reductions run in a fixed order
    base2 = torch.empty_like(base)
    x2, aux2 = base2[offset:offset + n], torch.zeros_like(aux)
    x2.copy_(y)
    lib.mxb_dp_finalize(_p(x2), n, 1.0 / 3.0, 2.0, _p(aux2, 4), _p(aux2, 1), None)
    assert torch.equal(aux2[1:4], aux[1:4])
    aux[3] = 0.25
    assert lib.mxb_dp_scale(_p(x), n, _p(aux, 3), None) == 0
    assert torch.equal(x, wanty * 0.25)


@pytest.mark.parametrize("den", [3.0, 0.0, float("nan")])
def test_finalize_with_device_denominator(den):
    """mxb_dp_finalize_dev reads the divisor from device memory: same bits as the host-argument form for a valid
    denominator; a zero or non-finite one leaves the values undivided (the host decides about the step)."""
    lib = mixlab_b200.lib()
    n = 100_003
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(n, device="cuda", generator=g)
    y = x.clone()
    d = torch.tensor([den], device="cuda")
    a1 = torch.zeros(4 + lib.mxb_dp_partial_floats(), device="cuda")
    a2 = torch.zeros_like(a1)
    assert lib.mxb_dp_finalize_dev(_p(x), n, _p(d), 2.0, _p(a1, 4), _p(a1, 1), None) == 0
    inv = 1.0 / den if den > 0 else 1.0
    inv32 = (torch.ones(1) / torch.tensor([den])).item() if den > 0 else 1.0   # the float32 reciprocal the kernel forms
    assert lib.mxb_dp_finalize(_p(y), n, inv32, 2.0, _p(a2, 4), _p(a2, 1), None) == 0
    assert torch.equal(x, y) and torch.equal(a1[1:4], a2[1:4])
    assert lib.mxb_dp_finalize_dev(_p(x), n, None, 2.0, _p(a1, 4), _p(a1, 1), None) != 0


def test_staged_step_on_one_rank_nccl_group():
    import torch.distributed as dist
    from mixlab_b200 import dp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE="1")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        shapes = [(300, 200), (200,), (1000, 64), (5,)]
        plan = dp.build_gradient_bucket_plan(shapes, target_bytes=100_000)
        g = torch.Generator().manual_seed(9)
        host = [torch.randn(*sh, generator=g) for sh in shapes]
        comm = torch.cuda.Stream()
        grads = [t.cuda() for t in host]
        res = dp.staged_gradient_allreduce(grads, torch.ones((), device="cuda"), 4.0, False, 1.5, plan, comm_stream=comm)
        norm = math.sqrt(sum(float(t.double().pow(2).sum()) for t in host))       # mean gradient = own gradient here
        scale = min(1.0, 1.5 / (norm + 1e-6))
        assert not res.globally_bad and not res.zero_denominator and res.denominator == 4.0 and res.gradient_nonfinite == 0.0
        for a, b in zip(grads, host):
            assert torch.allclose(a.cpu(), b * scale, rtol=1e-5, atol=1e-6)
        bad = [t.cuda() for t in host]
        bad[1][7] = float("nan")
        res = dp.staged_gradient_allreduce(bad, torch.ones((), device="cuda"), 4.0, False, 1.5, plan, comm_stream=comm)
        assert res.globally_bad
        res = dp.staged_gradient_allreduce([t.cuda() for t in host], torch.ones((), device="cuda"), 0.0, False, 0.0, plan)
        assert res.zero_denominator
    finally:
        dist.destroy_process_group()
