#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the reference's own code.

Run once in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's pure-Python / pure-torch implementations of the
scan primitives (never its compiled code), runs them on the reference's own
fixture inputs and on extra seeded inputs, and writes input/output vectors.
The tests only read the written files.

Sources used (paths inside the reference checkout):
  experiments/gated_deltanet_reference/generate_fixtures.py   scalar GDN block + scan
  experiments/mamba3_reference/generate_fixtures.py           scalar Mamba-3 block + scan
  experiments/gated_deltanet_test/dump_fla_reference_pure.py  torch GDN recurrence
  train/hf_templates/mamba3_mixlab.py                         torch Mamba-3 scan and full canonical block
  experiments/gated_deltanet_test/dump_fla_grad_reference.py  torch GDN full block, forward + every weight gradient
  train/testdata/gated_deltanet_full_block_reference.json     checked-in expected output
  train/testdata/mamba3_full_block_reference.json             checked-in expected output
  gpu/gated_delta_scan_test.go:44-83                          closed-form test inputs (restated below)
"""

from __future__ import annotations

import importlib.util
import json
import math
import random
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _record(mod, fn_name):
    calls = []
    orig = getattr(mod, fn_name)

    def wrapper(*a):
        r = orig(*a)
        calls.append((a, r))
        return r

    setattr(mod, fn_name, wrapper)
    return calls


def gdn_block_fixture(ref: Path):
    mod = _load(ref / "experiments/gated_deltanet_reference/generate_fixtures.py", "ref_gdn_fix")
    calls = _record(mod, "gated_delta_scan")
    fx = mod.fixture()
    checked = json.loads((ref / "train/testdata/gated_deltanet_full_block_reference.json").read_text())
    want = checked["fixtures"][0]["expected_hidden"]
    assert max(abs(a - b) for a, b in zip(fx["expected_hidden"], want)) < 1e-12, "generator != checked-in JSON"
    (a, r), = calls
    q, k, v, beta, gate, B, T, H, Dk, Dv = a
    cases = [dict(name="full_block_fixture_scan", B=B, T=T, H=H, Dk=Dk, Dv=Dv,
                  q=q, k=k, v=v, beta=beta, gate=gate, out=r,
                  source="scan call inside experiments/gated_deltanet_reference/generate_fixtures.py fixture(); "
                         "its block output equals train/testdata/gated_deltanet_full_block_reference.json")]
    # extra seeded cases through the same scalar reference loops
    rng = random.Random(1234)
    for (B, T, H, Dk, Dv) in [(2, 9, 2, 4, 5), (1, 70, 2, 8, 6), (1, 130, 1, 4, 4)]:
        def vec(n, lo=-1.0, hi=1.0):
            return [rng.uniform(lo, hi) for _ in range(n)]
        q = vec(B * T * H * Dk)
        k = vec(B * T * H * Dk)
        # normalise k per head vector so the recurrence stays bounded
        for i in range(B * T * H):
            nrm = math.sqrt(sum(x * x for x in k[i * Dk:(i + 1) * Dk])) or 1.0
            k[i * Dk:(i + 1) * Dk] = [x / nrm for x in k[i * Dk:(i + 1) * Dk]]
        v = vec(B * T * H * Dv)
        beta = vec(B * T * H, 0.05, 0.95)
        gate = vec(B * T * H, 0.3, 1.0)
        out = mod.gated_delta_scan(q, k, v, beta, gate, B, T, H, Dk, Dv)
        cases.append(dict(name=f"scalar_loops_B{B}_T{T}_H{H}_K{Dk}_V{Dv}", B=B, T=T, H=H, Dk=Dk, Dv=Dv,
                          q=q, k=k, v=v, beta=beta, gate=gate, out=out,
                          source="gated_delta_scan() of experiments/gated_deltanet_reference/generate_fixtures.py "
                                 "on python random.Random(1234) inputs"))
    (HERE / "gdn_scalar_reference.json").write_text(json.dumps(dict(cases=cases)))
    print("gdn_scalar_reference.json:", [c["name"] for c in cases])


def gdn_torch_recurrence(ref: Path):
    mod = _load(ref / "experiments/gated_deltanet_test/dump_fla_reference_pure.py", "ref_gdn_pure")
    g = torch.Generator().manual_seed(7)
    B, T, H, Dk, Dv = 2, 150, 3, 16, 24
    q = torch.randn(B, T, H, Dk, generator=g, dtype=torch.float64)
    k = torch.randn(B, T, H, Dk, generator=g, dtype=torch.float64)
    v = torch.randn(B, T, H, Dv, generator=g, dtype=torch.float64)
    q = q / q.norm(dim=-1, keepdim=True)
    k = k / k.norm(dim=-1, keepdim=True)
    beta = torch.sigmoid(torch.randn(B, T, H, generator=g, dtype=torch.float64))
    decay = torch.exp(-torch.nn.functional.softplus(torch.randn(B, T, H, generator=g, dtype=torch.float64)))
    out = mod.gated_delta_rule_recurrence(q, k, v, beta, decay)
    np.savez_compressed(HERE / "gdn_torch_recurrence.npz", q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        beta=beta.numpy(), gate=decay.numpy(), out=out.numpy())
    print("gdn_torch_recurrence.npz", tuple(out.shape))


def gdn_go_test_inputs():
    """Closed-form inputs of TestGatedDeltaScanChunkedMatchesNaiveForwardAndGrad
    (gpu/gated_delta_scan_test.go:44-83, :174-190): x and the six weights are
    sin/cos formulas; q,k,v,beta,gate are x @ w_i with sigmoid / exp(-softplus)."""
    B, T, H, dk, dv, dm, classes = 2, 97, 3, 8, 12, 16, 7
    shapes = [(dm, H * dk), (dm, H * dk), (dm, H * dv), (dm, H), (dm, H), (dv, classes)]
    ws = []
    for wi, (r, c) in enumerate(shapes):
        scale = np.float32(0.035 if wi in (2, 5) else 0.05)
        i = np.arange(r * c)
        angle = ((wi + 1) * (i % 17 + 1)).astype(np.float64)
        ws.append((scale * (np.sin(angle) * 0.7 + np.cos(angle * 0.37) * 0.3).astype(np.float32)).reshape(r, c))
    i = np.arange(B * T * dm)
    x = (np.float32(0.1) * (np.sin((i % 29).astype(np.float64)) * 0.6
                            + np.cos((i % 11).astype(np.float64)) * 0.4).astype(np.float32)).reshape(B * T, dm)
    x64 = x.astype(np.float64)
    q = (x64 @ ws[0]).reshape(B, T, H, dk)
    k = (x64 @ ws[1]).reshape(B, T, H, dk)
    v = (x64 @ ws[2]).reshape(B, T, H, dv)
    beta = 1.0 / (1.0 + np.exp(-(x64 @ ws[3]))).reshape(B, T, H)
    gate = np.exp(-np.log1p(np.exp(x64 @ ws[4]))).reshape(B, T, H)
    np.savez_compressed(HERE / "gdn_go_test_inputs.npz", q=q, k=k, v=v, beta=beta, gate=gate)
    print("gdn_go_test_inputs.npz", q.shape)


def mamba3_block_fixture(ref: Path):
    mod = _load(ref / "experiments/mamba3_reference/generate_fixtures.py", "ref_m3_fix")
    calls = _record(mod, "mamba3_scan")
    fx = mod.fixture()
    checked = json.loads((ref / "train/testdata/mamba3_full_block_reference.json").read_text())
    want = checked["fixtures"][0]["expected_hidden"]
    assert max(abs(a - b) for a, b in zip(fx["expected_hidden"], want)) < 1e-12, "generator != checked-in JSON"
    (a, r), = calls
    x, dt_raw, lam, theta, a_log, b, c, B, T, D, N, G = a
    cases = [dict(name="full_block_fixture_scan", B=B, T=T, D=D, N=N, G=G, x=x, dt_raw=dt_raw, lambda_raw=lam,
                  theta=theta, a_log=a_log, b=b, c=c, y=r,
                  source="scan call inside experiments/mamba3_reference/generate_fixtures.py fixture(); its block "
                         "output equals train/testdata/mamba3_full_block_reference.json")]
    (HERE / "mamba3_scalar_reference.json").write_text(json.dumps(dict(cases=cases)))
    print("mamba3_scalar_reference.json:", [c["name"] for c in cases])


def mamba3_torch_scan(ref: Path):
    mod = _load(ref / "train/hf_templates/mamba3_mixlab.py", "ref_m3_hf")
    out = {}
    for tag, (B, T, D, N, G, seed) in dict(a=(2, 8, 4, 8, 2, 11), b=(2, 37, 8, 16, 1, 12), c=(1, 20, 4, 128, 2, 13)).items():
        g = torch.Generator().manual_seed(seed)
        f64 = dict(generator=g, dtype=torch.float64)
        x = torch.randn(B, T, D, **f64)
        dt_raw = -1.0 + 0.7 * torch.randn(B, T, D, **f64)
        lam = torch.randn(B, T, D, **f64)
        theta = (2 * torch.rand(B, T, D, N // 2, **f64) - 1) * math.pi
        a_log = math.log(16.0) * torch.rand(D, N, **f64)
        b = torch.randn(B, T, G, N, **f64)
        c = torch.randn(B, T, G, N, **f64)
        fake = types.SimpleNamespace(state_size=N, inner_dim=D, n_groups=G, channels_per_group=D // G, A_log=a_log)
        mask = torch.ones(B, T, dtype=torch.bool)
        y = mod.MixlabMamba3CanonicalBlock._selective_scan(
            fake, x, dt_raw, lam, theta.reshape(B, T, D * (N // 2)), b.reshape(B, T, G * N), c.reshape(B, T, G * N), mask)
        for nme, t in dict(x=x, dt_raw=dt_raw, lambda_raw=lam, theta=theta, a_log=a_log, b=b, c=c, y=y).items():
            out[f"{tag}_{nme}"] = t.numpy()
    np.savez_compressed(HERE / "mamba3_torch_scan.npz", **out)
    print("mamba3_torch_scan.npz", sorted({k.split('_')[0] for k in out}))



def gdn_block_stages(ref: Path):
    """Pre- and post-scan stages of the gated_deltanet block (arch/blocks_gated_deltanet.go:207-343) through the
    reference's own scalar helpers (short_conv_1d, rms_norm_rows, silu, softplus, sigmoid of
    experiments/gated_deltanet_reference/generate_fixtures.py), on its fixture and on seeded inputs."""
    mod = _load(ref / "experiments/gated_deltanet_reference/generate_fixtures.py", "ref_gdn_fix2")
    rng = random.Random(4321)
    cases = []
    for (B, T, H, Dk, Dv) in [(1, 3, 1, 2, 3), (2, 7, 2, 8, 16), (1, 40, 3, 16, 8)]:
        def vec(n, lo=-1.0, hi=1.0):
            return [rng.uniform(lo, hi) for _ in range(n)]
        Ck, Cv = H * Dk, H * Dv
        qp, kp, vp = vec(B * T * Ck, -2, 2), vec(B * T * Ck, -2, 2), vec(B * T * Cv, -2, 2)
        wq, wk, wv = vec(4 * Ck, -0.5, 0.5), vec(4 * Ck, -0.5, 0.5), vec(4 * Cv, -0.5, 0.5)
        a_raw, b_raw = vec(B * T * H, -3, 3), vec(B * T * H, -3, 3)
        a_log, dt_bias = vec(H, -1, 1), vec(H, -0.5, 0.5)
        q_seq = mod.short_conv_1d(qp, wq, B, T, Ck)
        k_seq = mod.short_conv_1d(kp, wk, B, T, Ck)
        v_seq = mod.short_conv_1d(vp, wv, B, T, Cv)
        q_unit = mod.rms_norm_rows(q_seq, B * T * H, Dk, [1.0] * Dk, 1e-6)
        k_unit = mod.rms_norm_rows(k_seq, B * T * H, Dk, [1.0] * Dk, 1e-6)
        inv = 1.0 / math.sqrt(Dk)
        q = [x * inv * inv for x in q_unit]
        k = [x * inv for x in k_unit]
        gate, beta = [], []
        for i, x in enumerate(a_raw):
            h = i % H
            dt = mod.softplus(x + dt_bias[h])
            gate.append(math.exp(-dt * math.exp(a_log[h])))
        beta = [mod.sigmoid(x) for x in b_raw]
        # post stage
        o, z, onw = vec(B * T * H * Dv, -2, 2), vec(B * T * H * Dv, -3, 3), vec(Dv, 0.5, 1.5)
        y_norm = mod.rms_norm_rows(o, B * T * H, Dv, onw, 1e-5)
        y = [a * mod.silu(b) for a, b in zip(y_norm, z)]
        cases.append(dict(B=B, T=T, H=H, Dk=Dk, Dv=Dv, q_proj=qp, k_proj=kp, v_proj=vp, conv_q=wq, conv_k=wk, conv_v=wv,
                          a_raw=a_raw, b_raw=b_raw, a_log=a_log, dt_bias=dt_bias, q=q, k=k, v=v_seq, beta=beta, gate=gate,
                          o=o, z=z, o_norm=onw, y=y))
    (HERE / "gdn_block_stages.json").write_text(json.dumps(dict(
        cases=cases, source="helpers of experiments/gated_deltanet_reference/generate_fixtures.py composed as in "
                            "fixture() / arch/blocks_gated_deltanet.go:207-343, python random.Random(4321) inputs")))
    print("gdn_block_stages.json:", len(cases), "cases")


def mamba3_block_stages(ref: Path):
    """Element-wise stages of the canonical Mamba-3 block (gpu/ir.cpp:2034-2105) through the reference's own
    scalar helpers (depthwise_conv_1d, rms_norm_rows, sigmoid of experiments/mamba3_reference/generate_fixtures.py)."""
    mod = _load(ref / "experiments/mamba3_reference/generate_fixtures.py", "ref_m3_fix2")
    rng = random.Random(8765)
    cases = []
    for (B, T, D, N, G, K) in [(1, 3, 4, 2, 1, 4), (2, 9, 16, 8, 2, 4), (1, 37, 24, 16, 1, 3)]:
        def vec(n, lo=-1.0, hi=1.0):
            return [rng.uniform(lo, hi) for _ in range(n)]
        x, w = vec(B * T * D, -2, 2), vec(D * K, -0.6, 0.6)
        conv = mod.depthwise_conv_1d(x, w, B, T, D, K)
        bp, cp = vec(B * T * G * N, -2, 2), vec(B * T * G * N, -2, 2)
        bs, cs, bb, cb = vec(N, 0.5, 1.5), vec(N, 0.5, 1.5), vec(G * N, -0.5, 0.5), vec(G * N, -0.5, 0.5)
        bn = mod.rms_norm_rows(bp, B * T * G, N, bs)
        cn = mod.rms_norm_rows(cp, B * T * G, N, cs)
        b = [v + bb[i % (G * N)] for i, v in enumerate(bn)]
        c = [v + cb[i % (G * N)] for i, v in enumerate(cn)]
        y, z, pn = vec(B * T * D, -2, 2), vec(B * T * D, -3, 3), vec(D, 0.5, 1.5)
        yn = mod.rms_norm_rows(y, B * T, D, pn)
        out = [a * zz * mod.sigmoid(zz) for a, zz in zip(yn, z)]
        cases.append(dict(B=B, T=T, D=D, N=N, G=G, K=K, x=x, conv_w=w, conv=conv, b_proj=bp, c_proj=cp, b_scale=bs,
                          c_scale=cs, b_bias=bb, c_bias=cb, b=b, c=c, y=y, z=z, post_norm=pn, out=out))
    (HERE / "mamba3_block_stages.json").write_text(json.dumps(dict(
        cases=cases, source="helpers of experiments/mamba3_reference/generate_fixtures.py composed as in fixture() / "
                            "gpu/ir.cpp:2034-2105 (eps 1e-5), python random.Random(8765) inputs")))
    print("mamba3_block_stages.json:", len(cases), "cases")

def gdn_fla_grad_fixtures(ref: Path):
    """The reference's own gradient fixture of one full gated_deltanet block (ReferenceStack of
    dump_fla_reference_pure.py:94-155 driven by dump_fla_grad_reference.py, the generator behind
    train/gated_deltanet_fla_grad_parity_test.go): input, every weight, the block output and the gradient of
    mean(y^2) with respect to every weight, with and without kv_share, at the generator's default sizes."""
    sys.path.insert(0, str(ref / "experiments/gated_deltanet_test"))
    mod = _load(ref / "experiments/gated_deltanet_test/dump_fla_grad_reference.py", "ref_gdn_grad")
    for share in (True, False):
        cfg = mod.Config(model_dim=64, heads=4, d_k=8, d_v=16, seq_len=16, layers=1, kv_share=share, seed=7)
        name = "gdn_fla_grad_kvshare.npz" if share else "gdn_fla_grad_nokvshare.npz"
        mod.save_grad_fixture(str(HERE / name), cfg)


def mamba3_full_block_torch(ref: Path):
    """One canonical Mamba-3 block through the reference's own torch module (MixlabMamba3CanonicalBlock of
    train/hf_templates/mamba3_mixlab.py: pre-norm, projections, causal depthwise conv, B/C norm + bias, scan,
    post-norm x gate, output projection, residual) in float64: input, every parameter, the output and the gradient of
    mean(y^2) with respect to every parameter (torch autograd through the module's own code)."""
    mod = _load(ref / "train/hf_templates/mamba3_mixlab.py", "ref_m3_hf2")
    torch.manual_seed(21)
    cfg = types.SimpleNamespace(model_dim=32)
    blk = mod.MixlabMamba3CanonicalBlock(cfg, dict(inner_dim=32, state_size=16, n_groups=2, dt_rank=2, conv_kernel=4)).double()
    with torch.no_grad():  # the module's A_log is left uninitialised (torch.empty): give it the documented range
        blk.A_log.copy_(math.log(16.0) * torch.rand(32, 16, dtype=torch.float64))
        blk.dt_bias.copy_(-1.0 + 0.5 * torch.randn(32, dtype=torch.float64))
        for nrm in (blk.pre_norm, blk.B_norm, blk.C_norm, blk.post_norm):
            nrm.weight.copy_(1.0 + 0.2 * torch.randn_like(nrm.weight))
        blk.B_bias.copy_(1.0 + 0.3 * torch.randn_like(blk.B_bias))
        blk.C_bias.copy_(1.0 + 0.3 * torch.randn_like(blk.C_bias))
    B, T = 2, 24
    x = torch.randn(B, T, 32, dtype=torch.float64)
    y = blk(x)
    loss = y.pow(2).mean()
    loss.backward()
    out = dict(input=x.numpy(), output=y.detach().numpy(), loss=np.array([loss.item()]),
               dims=np.array([B, T, 32, 32, 16, 2, 2, 4], dtype=np.int64))  # B, T, model, inner, state, groups, rank, K
    for name, prm in blk.named_parameters():
        out["w:" + name] = prm.detach().numpy()
        out["g:" + name] = prm.grad.detach().numpy()
    np.savez_compressed(HERE / "mamba3_full_block_torch.npz", **out)
    print("mamba3_full_block_torch.npz", sorted(k for k in out if k.startswith("w:")))


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference-checkout")
    ref = Path(sys.argv[1])
    gdn_block_fixture(ref)
    gdn_block_stages(ref)
    gdn_torch_recurrence(ref)
    gdn_go_test_inputs()
    mamba3_block_fixture(ref)
    mamba3_block_stages(ref)
    mamba3_torch_scan(ref)
    gdn_fla_grad_fixtures(ref)
    mamba3_full_block_torch(ref)


if __name__ == "__main__":
    main()
