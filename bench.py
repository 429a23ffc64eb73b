#!/usr/bin/env python3
"""Benchmark of the B200 gated-delta / Mamba-3 kernels.

    python bench.py --gpus N --steps K --warmup W [--workload gdn_train|gdn_decode|mamba3_train]
    python bench.py --impl reference ...        # CPU arm: the oracle's restatement of the reference

One JSON line on stdout (rank 0).  Default workload = the configuration the
headline metric is quoted on: gated delta rule forward+backward, B=8 per GPU,
T=4096, H=16, d_k=d_v=128, chunk 64, bf16 I/O with fp32 state (seeded synthetic
inputs).  A step is one forward + one backward over that batch.  Multi-GPU runs
shard by batch (weak scaling) with no data-path collective.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: dims
    "gdn_train": dict(B=8, T=4096, H=16, Dk=128, Dv=128, chunk=64),
    "gdn_decode": dict(N=256, H=16, Dk=128, Dv=128, tokens_per_step=64),
    "mamba3_train": dict(B=8, T=4096, nheads=32, headdim=64, N=128, G=1),
    "gdn_block": dict(B=8, T=4096, H=16, Dk=128, Dv=128),
    "mamba3_block": dict(B=8, T=4096, D=2048, N=128, G=1, K=4),
    # the shape the reference's own scan benchmark is quoted on, in its per-channel float32 layout
    "mamba3_ref_shape": dict(B=2, T=1024, D=128, N=16, G=4),
}
# Algorithmic work per unit: the bytes that must cross HBM if every intermediate stayed on chip.
GDN_BYTES_PER_TOKEN_HEAD = 2840          # fwd 1032 + bwd read 1032 + bwd write 776
GDN_FLOPS_PER_TOKEN_HEAD = 3 * 182955    # fwd + 2x for bwd


def gdn_bytes_per_token_head(dk, dv, io_bytes=2):
    """fwd: q,k,v,o + beta,g fp32; bwd: q,k,v,dO,beta,g in, dq,dk,dv + dbeta,dg fp32 out (bf16 tensors unless io_bytes=4)."""
    e = io_bytes
    return e * (2 * dk + 2 * dv) + 8 + e * (2 * dk + 2 * dv) + 8 + e * (2 * dk + dv) + 8
M3_BYTES_PER_TOKEN = 23168
M3_FLOPS_PER_TOKEN = 5.50e6
# block stages around the scan, fwd+bwd, bf16: pre fwd 3 in + 3 out, pre bwd 6 in + 3 out, post fwd 2 in + 1 out,
# post bwd 3 in + 2 out = 23 tensors of 128 channels x 2 bytes, plus the fp32 per-head scalars
GDN_BLOCK_BYTES_PER_TOKEN_HEAD = 23 * 128 * 2 + 10 * 4
# Mamba-3 block stages, fwd+bwd, bf16: conv 2 + 3, post 3 + 5 tensors of D channels; B/C norm 4 + 6 tensors of G*N
M3_BLOCK_BYTES_PER_TOKEN = lambda D, GN: (13 * D + 10 * GN) * 2
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum, MB per launch at the full workload size) per kernel, from
# one ncu byte capture of a step.  Keyed by kernel name: when the kernels a step launches are not exactly these, the
# capture no longer describes the step and roofline.traffic is reported as null instead of a stale number.
GDN_NCU_TRAFFIC_MB = {   # captured at B=4 (4096 units); at B=8 a little less of the producer -> consumer tiles stays in L2
    "gdn_tc_prep_kernel": 353.9, "gdn_tc_state_fwd_kernel": 524.6, "gdn_tc_state_bwd_kernel": 464.9,
    "gdn_tc_chunk_bwd_kernel": 886.5,
}
GDN_NCU_TRAFFIC_UNITS = 4096     # (batch, head, chunk) units of the captured step
M3_NCU_TRAFFIC_MB = {
    "m3s_scalars_kernel": 12.6, "m3s_chunk_scalars_kernel": 12.6, "m3s_state_pass_kernel": 390.3 + 390.4,
    "m3s_chunk_out_kernel": 566.2, "m3s_chunk_grad_kernel": 1494.2, "m3s_final_kernel": 33.6, "m3s_dalog_kernel": 0.0,
    "m3s_reduce_kernel": 548.0,
}
M3_NCU_TRAFFIC_UNITS = 16384
DECODE_NCU_TRAFFIC_MB = {"gdn_decode_bulk_kernel": 482.8}
DECODE_NCU_TRAFFIC_UNITS = 4096  # (sequence, head) tiles of the captured launch


def traffic_from_table(table, table_units, units, kernels, launches_per_step=1):
    """Bytes per step from the per-kernel capture, or None when the step's kernel list differs from the capture's."""
    if not kernels or set(kernels) != set(table):
        return None
    return sum(table.values()) * 1e6 * launches_per_step * units / table_units


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm=float(d["hbm_gbs"]), tf_burst=float(d["bf16_tflops"]),
                    tf_sus=float(d["bf16_tflops_sustained"]), src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sus=1400.0, src="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for ts, line in self.rows:
            if ts < t0 or ts > t1 + 0.2:
                continue
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[0])); mx = float(f[1])
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:  # region shorter than one sample: take everything we saw
            for _, line in self.rows:
                f = [x.strip() for x in line.split(",")]
                try:
                    sm.append(float(f[0])); mx = float(f[1])
                except (ValueError, IndexError):
                    pass
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=mx, reasons=sorted(reasons),
                    samples=len(sm))


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ----------------------------------------------------------------------------- CPU arm
def cpu_gdn_sample(threads: int, passes: int):
    """Times the oracle's op-for-op restatement of gated_delta_scan_chunked (forward) plus
    torch autograd (backward; the reference uses MLX autograd) in fp32 on the host cores, on
    B=1 of the 8 sequences of the workload (4096 tokens x 16 heads)."""
    from oracle import gdn, inputs
    torch.set_num_threads(threads)
    w = WORKLOADS["gdn_train"]
    a = inputs.gdn_inputs(1, w["T"], w["H"], w["Dk"], w["Dv"], seed=1, io_dtype=torch.bfloat16, with_grad_out=True)
    f = {k: v.float() for k, v in a.items()}
    times = []
    for _ in range(passes):
        t = time.perf_counter()
        gdn.scan_grads(f["q"], f["k"], f["v"], f["beta"], f["g"], f["d_out"], gate_is_log=True, chunk_size=w["chunk"])
        times.append(time.perf_counter() - t)
    return w["T"], times


def gdn_train_cfg(w, world):
    """The config object of the headline workload (the same for both arms)."""
    return {"workload": "gdn_train", **w, "io": "bf16", "state": "fp32", "per_gpu_batch": w["B"],
            "parallelism": f"batch-sharded x{world}, no collective",
            "l2": "inputs (q,k,v,dO = 4 x 134 MB at B=8) exceed the 126 MB L2"}


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    tok, warm = cpu_gdn_sample(threads, max(1, min(args.warmup, 1)))
    tok, times = cpu_gdn_sample(threads, max(1, min(args.steps, 4)))
    dt = sum(times) / len(times)
    val = tok / dt
    w = WORKLOADS["gdn_train"]
    sample = f"B=1 of {w['B']} sequences (T={w['T']}, H={w['H']}, d={w['Dk']}), fp32, {len(times)} passes"
    print(json.dumps({
        "impl": "reference", "metric": "gdn_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": 1, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": gdn_train_cfg(w, max(1, args.gpus)),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------- GPU arm
class Ctx:
    """What the workload builders and the timing loop share."""

    def __init__(self, args):
        self.args = args
        self.rank, self.world, self.local = dist_env()
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            self.dist = dist
        import mixlab_b200
        from mixlab_b200 import ops, _lib, sharding
        from oracle import inputs  # seeded input generators only (no compute)
        self.mx, self.ops, self._lib, self.sharding, self.inputs = mixlab_b200, ops, _lib, sharding, inputs
        self.lib = mixlab_b200.lib()
        self.pk = peaks()

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()


def build_gdn_train(cx, batch):
    w = dict(WORKLOADS["gdn_train"])
    if batch > 0:
        w["B"] = batch
    if cx.args.dims:
        w["B"], w["T"], w["H"], w["Dk"], w["Dv"] = (int(x) for x in cx.args.dims.split(","))
    B, T, H, K, V, Cc = w["B"], w["T"], w["H"], w["Dk"], w["Dv"], w["chunk"]
    flags = cx._lib.MXB_GDN_FORCE_FP32_PATH if cx.args.fp32_path else 0
    f32 = cx.args.io == "f32"
    if f32 and not cx.args.fp32_path:  # float32 tensors, bf16 operands inside (the flag is off by default)
        flags |= cx._lib.MXB_GDN_F32_IO_BF16_OPERANDS
    # seeded inputs, generated one sequence at a time to bound host memory
    parts = [cx.inputs.gdn_inputs(1, T, H, K, V, seed=1000 * (cx.rank + 1) + b,
                                  io_dtype=torch.float32 if f32 else torch.bfloat16, with_grad_out=True) for b in range(B)]
    host = {k: torch.cat([p[k] for p in parts]).contiguous().pin_memory() for k in parts[0]}
    d = {k: v.to(cx.dev, non_blocking=True) for k, v in host.items()}
    units = B * T  # tokens per step per GPU
    ops = cx.ops

    def step():
        ops.gated_delta_scan(d["q"], d["k"], d["v"], d["beta"], d["g"], Cc, gate_is_log=True, flags=flags,
                             save_for_backward=True)
        ops.gated_delta_scan_backward(d["q"], d["k"], d["v"], d["beta"], d["g"], d["d_out"], Cc,
                                      gate_is_log=True, flags=flags, use_saved=True)

    nchunks = B * H * ((T + Cc - 1) // Cc)
    cfg = gdn_train_cfg(w, cx.world)
    if f32:
        cfg["io"] = "f32 tensors" + (", fp32 kernels" if cx.args.fp32_path else ", bf16 operands inside (MXB_GDN_F32_IO_BF16_OPERANDS)")
    return dict(step=step, units=units, metric="gdn_fwd_bwd_tokens_per_s", unit="tokens/s",
                dtype="f32" if (f32 and cx.args.fp32_path) else "bf16",
                alg_bytes=units * H * gdn_bytes_per_token_head(K, V, 4 if f32 else 2),
                alg_flops=units * H * GDN_FLOPS_PER_TOKEN_HEAD * (K * V) / (128.0 * 128.0),
                traffic=(lambda kernels: traffic_from_table(GDN_NCU_TRAFFIC_MB, GDN_NCU_TRAFFIC_UNITS, nchunks, kernels))
                if (K, V) == (128, 128) and not f32 else (lambda kernels: None),
                traffic_note="per-kernel ncu byte capture (dram bytes read + written) of a full-size step, scaled by the "
                             "number of (batch, head, chunk) units; null when the step's kernel list differs from the capture's",
                cfg=cfg, host=host, dev_tensors=d, w=w, flags=flags)


def build_gdn_decode(cx, batch):
    w = dict(WORKLOADS["gdn_decode"])
    if batch > 0:
        w["N"] = batch
    N, H, K, V, tps = w["N"], w["H"], w["Dk"], w["Dv"], w["tokens_per_step"]
    a = cx.inputs.gdn_decode_inputs(N, H, K, V, 16, seed=2 + cx.rank, io_dtype=torch.bfloat16)
    d = {k: v.to(cx.dev) for k, v in a.items()}
    out = torch.empty(N, H, V, dtype=torch.bfloat16, device=cx.dev)
    units = N * tps
    per_tok_bytes = 2 * K * V * 4 * H + (2 * K + 2 * V) * 2 * H + 8 * H
    ops = cx.ops

    def step():
        for t in range(tps):
            i = t % 16
            ops.gated_delta_decode_step(d["state"], d["q"][i], d["k"][i], d["v"][i], d["beta"][i], d["g"][i],
                                        gate_is_log=True, out=out)

    return dict(step=step, units=units, metric="gdn_decode_tokens_per_s", unit="tokens/s", dtype="f32",
                alg_bytes=units * per_tok_bytes, alg_flops=units * H * 7 * K * V,
                traffic=lambda kernels: traffic_from_table(DECODE_NCU_TRAFFIC_MB, DECODE_NCU_TRAFFIC_UNITS, N * H, kernels,
                                                           launches_per_step=tps) if (K, V) == (128, 128) else None,
                traffic_note="ncu byte capture of one launch at config 2, scaled by the (sequence, head) tiles and the "
                             "launches per step",
                cfg={"workload": "gdn_decode", **w, "io": "bf16", "state": "fp32 268 MB at N=256 (exceeds L2)",
                     "inputs": "ring of 16 pre-generated token inputs"})


def build_gdn_block(cx, batch):
    w = dict(WORKLOADS["gdn_block"])
    if batch > 0:
        w["B"] = batch
    B, T, H, K, V = w["B"], w["T"], w["H"], w["Dk"], w["Dv"]
    g = torch.Generator().manual_seed(4000 + cx.rank)
    rn = lambda *shape: torch.randn(*shape, generator=g)
    io = torch.bfloat16
    d = dict(qp=rn(B, T, H * K).to(io), kp=rn(B, T, H * K).to(io), vp=rn(B, T, H * V).to(io),
             cq=0.4 * rn(4, H * K), ck=0.4 * rn(4, H * K), cv=0.4 * rn(4, H * V), a=rn(B, T, H), b=rn(B, T, H),
             al=0.5 * rn(H), bias=0.3 * rn(H), o=rn(B, T, H, V).to(io), z=rn(B, T, H * V).to(io), wn=1 + 0.2 * rn(V),
             dq=rn(B, T, H, K).to(io), dk=rn(B, T, H, K).to(io), dv=rn(B, T, H, V).to(io), db=rn(B, T, H),
             dg=rn(B, T, H), dy=rn(B, T, H * V).to(io))
    d = {k: v.to(cx.dev) for k, v in d.items()}
    units = B * T
    pre = [d[k] for k in ("qp", "kp", "vp", "cq", "ck", "cv", "a", "b", "al", "bias")]
    ops = cx.ops

    def step():
        ops.gdn_block_pre(*pre, H, K, V, gate_is_log=True)
        ops.gdn_block_post(d["o"], d["z"], d["wn"])
        ops.gdn_block_post_backward(d["o"], d["z"], d["wn"], d["dy"])
        ops.gdn_block_pre_backward(*pre, H, K, V, d["dq"], d["dk"], d["dv"], d["db"], d["dg"], gate_is_log=True)

    return dict(step=step, units=units, metric="gdn_block_stages_fwd_bwd_tokens_per_s", unit="tokens/s", dtype="f32",
                alg_bytes=units * H * GDN_BLOCK_BYTES_PER_TOKEN_HEAD, alg_flops=0.0, traffic=lambda kernels: None,
                traffic_note="not captured",
                cfg={"workload": "gdn_block", **w, "io": "bf16",
                     "what": "conv+SiLU+L2-norm/gate/beta and norm x gate, fwd+bwd"})


def build_mamba3_block(cx, batch):
    w = dict(WORKLOADS["mamba3_block"])
    if batch > 0:
        w["B"] = batch
    B, T, D, N, G, K = w["B"], w["T"], w["D"], w["N"], w["G"], w["K"]
    g = torch.Generator().manual_seed(5000 + cx.rank)
    rn = lambda *shape: torch.randn(*shape, generator=g)
    io = torch.bfloat16
    d = dict(x=rn(B, T, D).to(io), cw=0.4 * rn(D, K), dyc=rn(B, T, D).to(io),
             bp=rn(B, T, G * N).to(io), cp=rn(B, T, G * N).to(io), bs=1 + 0.2 * rn(N), cs=1 + 0.2 * rn(N),
             bb=0.3 * rn(G * N), cb=0.3 * rn(G * N), db=rn(B, T, G, N).to(io), dc=rn(B, T, G, N).to(io),
             y=rn(B, T, D).to(io), z=rn(B, T, D).to(io), pn=1 + 0.2 * rn(D), dout=rn(B, T, D).to(io))
    d = {k: v.to(cx.dev) for k, v in d.items()}
    units = B * T
    ops = cx.ops

    def step():
        ops.mamba3_block_conv(d["x"], d["cw"])
        ops.mamba3_block_bc(d["bp"], d["cp"], d["bs"], d["cs"], d["bb"], d["cb"], G, N)
        ops.mamba3_block_post(d["y"], d["z"], d["pn"])
        ops.mamba3_block_post_backward(d["y"], d["z"], d["pn"], d["dout"])
        ops.mamba3_block_bc_backward(d["bp"], d["cp"], d["bs"], d["cs"], d["db"], d["dc"], G, N)
        ops.mamba3_block_conv_backward(d["x"], d["cw"], d["dyc"])

    return dict(step=step, units=units, metric="mamba3_block_stages_fwd_bwd_tokens_per_s", unit="tokens/s", dtype="f32",
                alg_bytes=units * M3_BLOCK_BYTES_PER_TOKEN(D, G * N), alg_flops=0.0, traffic=lambda kernels: None,
                traffic_note="not captured",
                cfg={"workload": "mamba3_block", **w, "io": "bf16",
                     "what": "depthwise conv, B/C norm + bias, post-norm x gate, fwd+bwd"})


def build_mamba3_train(cx, batch):
    w = dict(WORKLOADS["mamba3_train"])
    if batch > 0:
        w["B"] = batch
    B, T, NH, P, N, G = w["B"], w["T"], w["nheads"], w["headdim"], w["N"], w["G"]
    parts = [cx.inputs.mamba3_inputs(1, T, NH, P, N, G=G, seed=3000 * (cx.rank + 1) + b, io_dtype=torch.bfloat16)
             for b in range(B)]
    keys = ("x", "dt_raw", "lambda_raw", "theta", "b", "c", "dy")
    d = {k: torch.cat([p[k] for p in parts]).to(cx.dev) for k in keys}
    d["a_log"] = parts[0]["a_log"].to(cx.dev)
    units = B * T
    margs = [d[k] for k in ("x", "dt_raw", "lambda_raw", "theta", "a_log", "b", "c")]
    ops = cx.ops

    def step():
        ops.mamba3_selective_scan(*margs, nheads=NH, save_for_backward=True)
        ops.mamba3_selective_scan_backward(*margs, d["dy"], nheads=NH, use_saved=True)

    nchunks = B * NH * ((T + 63) // 64)
    return dict(step=step, units=units, metric="mamba3_fwd_bwd_tokens_per_s", unit="tokens/s", dtype="bf16",
                alg_bytes=units * M3_BYTES_PER_TOKEN, alg_flops=units * M3_FLOPS_PER_TOKEN,
                traffic=lambda kernels: traffic_from_table(M3_NCU_TRAFFIC_MB, M3_NCU_TRAFFIC_UNITS, nchunks, kernels)
                if (P, N) == (64, 128) else None,
                traffic_note="per-kernel ncu byte capture (dram bytes read + written) of a full-size step, scaled by the "
                             "number of (batch, head, chunk) units; null when the step's kernel list differs from the capture's",
                cfg={"workload": "mamba3_train", **w, "io": "bf16", "layout": "head-broadcast dt/lambda/theta/a_log"})


def build_mamba3_ref_shape(cx, batch):
    w = dict(WORKLOADS["mamba3_ref_shape"])
    if batch > 0:
        w["B"] = batch
    B, T, D, N, G = w["B"], w["T"], w["D"], w["N"], w["G"]
    a = cx.inputs.mamba3_inputs(B, T, D, 1, N, G=G, seed=4000 + cx.rank, per_head=False)
    d = {k: a[k].to(cx.dev) for k in ("x", "dt_raw", "lambda_raw", "theta", "a_log", "b", "c", "dy")}
    margs = [d[k] for k in ("x", "dt_raw", "lambda_raw", "theta", "a_log", "b", "c")]
    ops = cx.ops

    def step():
        ops.mamba3_selective_scan(*margs)
        ops.mamba3_selective_scan_backward(*margs, d["dy"])

    # fp32: forward reads x, dt, lambda [D], theta [D N/2], B, C [G N] and writes y; the backward reads those and
    # dy and writes dx, ddt, dlambda, dtheta, dB, dC
    per_token = 4 * ((D * (4 + N // 2) + 2 * G * N) + (D * (4 + N // 2) + 2 * G * N) + (D * (3 + N // 2) + 2 * G * N))
    return dict(step=step, units=B * T, metric="mamba3_fwd_bwd_tokens_per_s", unit="tokens/s", dtype="f32",
                alg_bytes=B * T * per_token, alg_flops=0.0, traffic=lambda kernels: None,
                traffic_note="no byte capture for this workload (7 MB of tensors: it lives in L2)",
                cfg={"workload": "mamba3_ref_shape", **w, "io": "f32", "layout": "per-channel dt/lambda/theta/a_log (the reference's)",
                     "l2": "the whole problem fits L2; the step is bound by the T-long serial walk, not by HBM"})


BUILDERS = {"mamba3_ref_shape": build_mamba3_ref_shape, "gdn_train": build_gdn_train, "gdn_decode": build_gdn_decode, "gdn_block": build_gdn_block,
            "mamba3_block": build_mamba3_block, "mamba3_train": build_mamba3_train}


def time_workload(cx, wl, steps, warmup):
    """W warm-up steps, then exactly K steps between two barriers; device time by CUDA events (max over ranks), every
    kernel of the library timed by its own event pair on the launching stream, clocks sampled during the region."""
    lib, step = cx.lib, wl["step"]
    for _ in range(warmup):
        step()
    cx.barrier()
    sampler = ClockSampler(cx.local)
    sampler.start()
    time.sleep(0.25)
    lib.mxb_trace_enable(1)
    n0 = lib.mxb_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cx.barrier()
    t_wall0 = time.time()
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    cx.barrier()
    t_wall1 = time.time()
    ms = ev0.elapsed_time(ev1)
    launches = int(lib.mxb_launch_count() - n0)
    buf = C.create_string_buffer(1 << 16)
    lib.mxb_trace_summary(buf, len(buf))
    lib.mxb_trace_enable(0)
    clocks = sampler.stop(t_wall0, t_wall1)
    ms = cx.sharding.max_over_ranks(ms, cx.dev)
    kernels = {}
    for line in buf.value.decode().splitlines():
        name, cnt, tot = line.split()
        kernels[name] = dict(launches=int(cnt), total_ms=float(tot))
    ksum = sum(k["total_ms"] for k in kernels.values()) or 1.0
    for k in kernels.values():
        k["share"] = k["total_ms"] / ksum
        k["avg_ms"] = k["total_ms"] / max(k["launches"], 1)
    top = max(kernels, key=lambda n: kernels[n]["total_ms"]) if kernels else None
    ms_step = ms / steps
    value = cx.sharding.whole_job_rate(wl["units"], cx.world, ms_step * 1e-3)
    # roofline of the step, taken as one launch: algorithmic bytes / summed kernel time
    kern_ms_step = ksum / steps
    achieved = wl["alg_bytes"] / (kern_ms_step * 1e-3) / 1e9
    pk = cx.pk
    tfl = wl["alg_flops"] / (kern_ms_step * 1e-3) / 1e12
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s", "frac": achieved / pk["hbm"],
                "traffic": wl["traffic"](kernels), "traffic_note": wl["traffic_note"], "peak_source": pk["src"],
                "scope": "all kernels of one step (algorithmic bytes of the step / summed kernel time)",
                "top_kernel": top, "kernels": kernels, "tensor_tflops": tfl,
                "tensor_frac_of_sustained": tfl / pk["tf_sus"]}
    return dict(ms_step=ms_step, value=value, launches=launches, clocks=clocks, roofline=roofline)


def dp_allreduce_leg(cx, steps=5, warmup=2):
    """The gradient exchange of the end-to-end training configuration (12 layers, d_model 1024, vocab 32768: about
    1.07 GB of fp32 gradients) on this job's ranks: bucket plan of 32 MiB buckets, staged all-reduce (the loss
    denominator rides behind the first bucket, the bad flag behind the last; every bucket is finalized behind its own
    sum), NCCL on a communication stream.  Reports the whole staged step and
    the all-reduces alone; bus bandwidth = 2 (N-1)/N x bytes / time."""
    import torch.distributed as dist
    from mixlab_b200 import dp
    plan = dp.build_gradient_bucket_plan(dp.hybrid_lm_weight_shapes())
    store = dp.BucketStorage(plan, cx.dev)
    g = torch.Generator(device=cx.dev).manual_seed(7 + cx.rank)
    for buf in store.flat:
        buf.normal_(generator=g)
    comm = torch.cuda.Stream(cx.dev)
    loss = torch.ones((), device=cx.dev)

    def staged():
        grads = list(store.views)
        return dp.staged_gradient_allreduce(grads, loss, 1.0, True, 1.0, plan, storage=store, comm_stream=comm)

    def bare():
        works = [dist.all_reduce(buf, async_op=True) for buf in store.flat]
        for w in works:
            w.wait()

    out = {}
    for name, fn in (("staged_step", staged), ("allreduce_only", bare)):
        for _ in range(warmup):
            fn()
            for buf in store.flat:   # keep the values bounded across repeated sums
                buf.mul_(1.0 / cx.world)
        cx.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        cx.barrier()
        ms = cx.sharding.max_over_ranks(ev0.elapsed_time(ev1) / steps, cx.dev)
        nbytes = sum(b.numel() * 4 for b in store.flat)
        out[name] = {"ms": ms, "bus_gbs": 2.0 * (cx.world - 1) / cx.world * nbytes / (ms * 1e-3) / 1e9,
                     "alg_gbs": nbytes / (ms * 1e-3) / 1e9}
    out.update(bytes=plan.total_bytes, buckets=len(plan.buckets), bucket_target_bytes=plan.target_bytes,
               plan_digest=f"{plan.digest:016x}", n_ranks=cx.world,
               reference_points="measured on this pool: 8-rank all-reduce bus bandwidth 725 GB/s at 1 GiB, peer copy 770 GB/s")
    del store
    torch.cuda.empty_cache()
    return out


def copy_floor(cx, host, res, steps):
    """The host<->device traffic of one end-to-end step and nothing else: every input tensor uploaded by one
    cudaMemcpyAsync each on one stream while every result tensor is downloaded on a second stream (pinned host
    memory, no kernels), all ranks at once between the same barriers.  The end-to-end call cannot be faster."""
    up, down = torch.cuda.Stream(cx.dev), torch.cuda.Stream(cx.dev)
    names_in = ("q", "k", "v", "beta", "g", "d_out")
    dev_in = {k: torch.empty_like(host[k], device=cx.dev) for k in names_in}
    dev_out = {k: torch.empty_like(v, device=cx.dev) for k, v in res.items()}

    def once():
        with torch.cuda.stream(up):
            for k in names_in:
                dev_in[k].copy_(host[k], non_blocking=True)
        with torch.cuda.stream(down):
            for k, v in res.items():
                v.copy_(dev_out[k], non_blocking=True)
        up.synchronize()
        down.synchronize()

    once()
    cx.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        once()
    cx.barrier()
    dt = (time.perf_counter() - t0) / steps
    return cx.sharding.max_over_ranks(dt, cx.dev) * 1e3


def end_to_end_gdn(cx, wl):
    """The same step through the host-buffer C ABI (mxb_host_gdn): pinned host tensors in and out, blocking."""
    lib, mx, host, w = cx.lib, cx.mx, wl["host"], wl["w"]
    B, T, H, K, V, Cc = w["B"], w["T"], w["H"], w["Dk"], w["Dv"], w["chunk"]
    ctx = C.c_void_p()
    desc = mx.GdnDesc(B, T, H, K, V, Cc, mx.MXB_BF16, 1, wl["flags"])
    need = lib.mxb_gdn_bwd_workspace_bytes(C.byref(desc)) + 12 * B * T * H * max(K, V) * 2 + (64 << 20)
    wl["dev_tensors"].clear()
    torch.cuda.empty_cache()
    st = lib.mxb_host_ctx_create(cx.local, need, C.byref(ctx))
    if st != 0:
        return {"value": None, "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "error": f"mxb_host_ctx_create status {st}"}
    res = {n: torch.empty_like(host[s]).pin_memory() for n, s in
           (("out", "v"), ("dq", "q"), ("dk", "k"), ("dv", "v"), ("dbeta", "beta"), ("dgate", "g"))}
    p = lambda t: C.c_void_p(t.data_ptr())

    def host_step():
        s = lib.mxb_host_gdn(ctx, C.byref(desc), p(host["q"]), p(host["k"]), p(host["v"]), p(host["beta"]),
                             p(host["g"]), p(res["out"]), p(host["d_out"]), p(res["dq"]), p(res["dk"]),
                             p(res["dv"]), p(res["dbeta"]), p(res["dgate"]))
        if s != 0:
            raise RuntimeError(f"mxb_host_gdn status {s}")

    host_step()
    nst = max(2, min(cx.args.steps, 5))
    cx.barrier()
    t0 = time.perf_counter()
    for _ in range(nst):
        host_step()  # blocking: H2D + kernels + D2H + stream sync
    cx.barrier()
    dt = (time.perf_counter() - t0) / nst
    dt = cx.sharding.max_over_ranks(dt, cx.dev)
    lib.mxb_host_ctx_destroy(ctx)
    floor_ms = copy_floor(cx, host, res, nst)
    h2d = sum(host[k].numel() * host[k].element_size() for k in ("q", "k", "v", "beta", "g", "d_out"))
    d2h = sum(t.numel() * t.element_size() for t in res.values())
    return {"value": cx.world * wl["units"] / dt, "unit": wl["unit"], "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": dt * 1e3, "copy_floor_ms": floor_ms, "frac_of_copy_floor": floor_ms / (dt * 1e3),
            "copy_floor_note": "the same bytes by bare cudaMemcpyAsync on two streams, no kernels, all ranks at once",
            "api": "mxb_host_gdn (pinned host buffers, blocking)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gdn_train", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the short legs of the other workloads (decode, Mamba-3, block stages)")
    ap.add_argument("--fp32-path", action="store_true", help="force the CUDA-core fp32 kernels")
    ap.add_argument("--io", default="bf16", choices=["bf16", "f32"],
                    help="gdn_train only: float32 tensors (side measurement; the headline is bf16)")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the per-GPU batch (sequences) - small cases for profiler captures only")
    ap.add_argument("--dims", default="", help="gdn_train only: B,T,H,Dk,Dv of another shape (side measurements; the "
                                               "headline workload is the default)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference_arm(args)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU fallback")
    rank, world, local = dist_env()
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        # NCCL prints its version banner on stdout at VERSION level; stdout carries only the JSON line
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cx = Ctx(args)

    wl = BUILDERS[args.workload](cx, args.batch)
    main_res = time_workload(cx, wl, args.steps, args.warmup)

    # ---- short legs of the other two primitives the headline metric names (default workload only) ----
    extra = None
    if args.workload == "gdn_train" and not args.no_extra and args.batch == 0 and not args.dims:
        extra = {}
        for name, nsteps in (("gdn_decode", 3), ("mamba3_train", 5), ("mamba3_ref_shape", 5), ("gdn_block", 3),
                             ("mamba3_block", 3)):
            w2 = BUILDERS[name](cx, 0)
            r = time_workload(cx, w2, nsteps, 3)
            rf = r["roofline"]
            extra[name] = {"metric": w2["metric"], "value": r["value"], "unit": w2["unit"], "ms_per_step": r["ms_step"],
                           "steps": nsteps, "warmup": 3, "config": w2["cfg"], "clocks": r["clocks"],
                           "gpu_launches": r["launches"],
                           "roofline": {k: rf[k] for k in ("bound", "achieved", "peak", "unit", "frac", "traffic",
                                                           "top_kernel", "peak_source")},
                           "kernels": {n: {"launches": k["launches"], "avg_ms": k["avg_ms"], "share": k["share"]}
                                       for n, k in rf["kernels"].items()}}
            if name == "gdn_decode":  # one launch per token: the per-launch figure is the decode roofline
                tps = w2["cfg"]["tokens_per_step"]
                extra[name]["hbm_gbs_per_launch"] = w2["alg_bytes"] / tps / (rf["kernels"][rf["top_kernel"]]["avg_ms"] * 1e-3) / 1e9
            del w2
            torch.cuda.empty_cache()

    if extra is not None and world > 1:
        extra["dp_allreduce"] = dp_allreduce_leg(cx)

    e2e = None
    if args.workload == "gdn_train" and not args.no_e2e and not args.dims:
        e2e = end_to_end_gdn(cx, wl)

    cpu = None
    if rank == 0 and world == 1 and args.workload == "gdn_train" and not args.no_cpu_baseline and not args.dims:
        threads = os.cpu_count() or 1
        tok, times = cpu_gdn_sample(threads, 2)
        cpu = {"value": tok / (sum(times) / len(times)), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"B=1 of 8 sequences (T=4096, H=16, d=128), fp32, {len(times)} passes of "
                         "oracle.gdn.scan_chunked + torch autograd"}

    if rank == 0:
        line = {
            "metric": wl["metric"], "value": main_res["value"], "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": main_res["ms_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic", "config": wl["cfg"],
            "clocks": main_res["clocks"], "e2e": e2e, "gpu_launches": main_res["launches"],
            "roofline": main_res["roofline"], "cpu_baseline": cpu,
        }
        if extra is not None:
            line["extra"] = extra
        print(json.dumps(line))
    if world > 1:
        cx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
