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
}
# Algorithmic work per unit: the bytes that must cross HBM if every intermediate stayed on chip.
GDN_BYTES_PER_TOKEN_HEAD = 2840          # fwd 1032 + bwd read 1032 + bwd write 776
GDN_FLOPS_PER_TOKEN_HEAD = 3 * 182955    # fwd + 2x for bwd
M3_BYTES_PER_TOKEN = 23168
M3_FLOPS_PER_TOKEN = 5.50e6
# block stages around the scan, fwd+bwd, bf16: pre fwd 3 in + 3 out, pre bwd 6 in + 3 out, post fwd 2 in + 1 out,
# post bwd 3 in + 2 out = 23 tensors of 128 channels x 2 bytes, plus the fp32 per-head scalars
GDN_BLOCK_BYTES_PER_TOKEN_HEAD = 23 * 128 * 2 + 10 * 4
# Mamba-3 block stages, fwd+bwd, bf16: conv 2 + 3, post 3 + 5 tensors of D channels; B/C norm 4 + 6 tensors of G*N
M3_BLOCK_BYTES_PER_TOKEN = lambda D, GN: (13 * D + 10 * GN) * 2
# DRAM traffic per unit from the committed ncu captures (profiles/): dram__bytes_read.sum + dram__bytes_write.sum
GDN_NCU_TRAFFIC_PER_CHUNK = 5648.3e6 / 8192    # one-pass DRAM-byte capture of a full-size step: 5648.3 MB over 8 x 16 x 64 (batch, head, chunk) units
M3_NCU_TRAFFIC_PER_CHUNK = 3447.8e6 / 16384    # one-pass DRAM-byte capture of a full-size step: 3447.8 MB over 8 x 32 x 64 units
DECODE_NCU_TRAFFIC_PER_TILE = 482.8e6 / 4096   # full-size capture: 482.8 MB over 256 x 16 (sequence, head) tiles


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
        "config": {"workload": "gdn_train B=8/GPU T=4096 H=16 dk=dv=128 chunk=64 (CPU arm: bounded sample)", **w},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gdn_train", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--fp32-path", action="store_true", help="force the CUDA-core fp32 kernels")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the per-GPU batch (sequences) - small cases for profiler captures only")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference_arm(args)

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        # NCCL prints its version banner on stdout at VERSION level; stdout carries only the JSON line
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)

    import mixlab_b200
    from mixlab_b200 import ops, _lib, sharding
    from oracle import inputs  # seeded input generators only (no compute)
    lib = mixlab_b200.lib()
    pk = peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    flags = _lib.MXB_GDN_FORCE_FP32_PATH if args.fp32_path else 0
    e2e = None
    if args.workload == "gdn_train":
        w = dict(WORKLOADS["gdn_train"])
        if args.batch > 0:
            w["B"] = args.batch
        B, T, H, K, V, Cc = w["B"], w["T"], w["H"], w["Dk"], w["Dv"], w["chunk"]
        # seeded inputs, generated one sequence at a time to bound host memory
        parts = [inputs.gdn_inputs(1, T, H, K, V, seed=1000 * (rank + 1) + b, io_dtype=torch.bfloat16,
                                   with_grad_out=True) for b in range(B)]
        host = {k: torch.cat([p[k] for p in parts]).contiguous().pin_memory() for k in parts[0]}
        d = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
        units = B * T  # tokens per step per GPU
        metric, unit, dtype = "gdn_fwd_bwd_tokens_per_s", "tokens/s", "bf16"
        alg_bytes = units * H * GDN_BYTES_PER_TOKEN_HEAD
        alg_flops = units * H * GDN_FLOPS_PER_TOKEN_HEAD
        bound = "hbm"
        traffic = B * H * ((T + Cc - 1) // Cc) * GDN_NCU_TRAFFIC_PER_CHUNK if not args.fp32_path else None
        traffic_note = "one-pass ncu capture (dram bytes read + written) of a full-size step, per (batch, head, chunk) unit x units"

        def step():
            ops.gated_delta_scan(d["q"], d["k"], d["v"], d["beta"], d["g"], Cc, gate_is_log=True, flags=flags,
                                 save_for_backward=True)
            ops.gated_delta_scan_backward(d["q"], d["k"], d["v"], d["beta"], d["g"], d["d_out"], Cc,
                                          gate_is_log=True, flags=flags, use_saved=True)

        cfg = {"workload": "gdn_train", **w, "io": "bf16", "state": "fp32", "per_gpu_batch": B,
               "parallelism": f"batch-sharded x{world}, no collective",
               "l2": "inputs (q,k,v,dO = 4 x 134 MB) exceed the 126 MB L2"}
    elif args.workload == "gdn_decode":
        w = dict(WORKLOADS["gdn_decode"])
        if args.batch > 0:
            w["N"] = args.batch
        N, H, K, V, tps = w["N"], w["H"], w["Dk"], w["Dv"], w["tokens_per_step"]
        a = inputs.gdn_decode_inputs(N, H, K, V, 16, seed=2 + rank, io_dtype=torch.bfloat16)
        d = {k: v.to(dev) for k, v in a.items()}
        out = torch.empty(N, H, V, dtype=torch.bfloat16, device=dev)
        units = N * tps
        metric, unit, dtype = "gdn_decode_tokens_per_s", "tokens/s", "f32"
        per_tok_bytes = 2 * K * V * 4 * H + (2 * K + 2 * V) * 2 * H + 8 * H
        alg_bytes = units * per_tok_bytes
        alg_flops = units * H * 7 * K * V
        bound = "hbm"
        traffic = tps * N * H * DECODE_NCU_TRAFFIC_PER_TILE if (K, V) == (128, 128) else None
        traffic_note = "ncu capture of one launch at config 2, per launch x launches per step"

        def step():
            for t in range(tps):
                i = t % 16
                ops.gated_delta_decode_step(d["state"], d["q"][i], d["k"][i], d["v"][i], d["beta"][i], d["g"][i],
                                            gate_is_log=True, out=out)

        cfg = {"workload": "gdn_decode", **w, "io": "bf16", "state": "fp32 268 MB (exceeds L2)",
               "inputs": "ring of 16 pre-generated token inputs"}
    elif args.workload == "gdn_block":
        w = dict(WORKLOADS["gdn_block"])
        if args.batch > 0:
            w["B"] = args.batch
        B, T, H, K, V = w["B"], w["T"], w["H"], w["Dk"], w["Dv"]
        g = torch.Generator().manual_seed(4000 + rank)
        rn = lambda *shape: torch.randn(*shape, generator=g)
        io = torch.bfloat16
        d = dict(qp=rn(B, T, H * K).to(io), kp=rn(B, T, H * K).to(io), vp=rn(B, T, H * V).to(io),
                 cq=0.4 * rn(4, H * K), ck=0.4 * rn(4, H * K), cv=0.4 * rn(4, H * V), a=rn(B, T, H), b=rn(B, T, H),
                 al=0.5 * rn(H), bias=0.3 * rn(H), o=rn(B, T, H, V).to(io), z=rn(B, T, H * V).to(io), wn=1 + 0.2 * rn(V),
                 dq=rn(B, T, H, K).to(io), dk=rn(B, T, H, K).to(io), dv=rn(B, T, H, V).to(io), db=rn(B, T, H),
                 dg=rn(B, T, H), dy=rn(B, T, H * V).to(io))
        d = {k: v.to(dev) for k, v in d.items()}
        units = B * T
        metric, unit, dtype = "gdn_block_stages_fwd_bwd_tokens_per_s", "tokens/s", "f32"
        alg_bytes = units * H * GDN_BLOCK_BYTES_PER_TOKEN_HEAD
        alg_flops = 0.0
        bound = "hbm"
        traffic, traffic_note = None, "not captured"
        pre = [d[k] for k in ("qp", "kp", "vp", "cq", "ck", "cv", "a", "b", "al", "bias")]

        def step():
            ops.gdn_block_pre(*pre, H, K, V, gate_is_log=True)
            ops.gdn_block_post(d["o"], d["z"], d["wn"])
            ops.gdn_block_post_backward(d["o"], d["z"], d["wn"], d["dy"])
            ops.gdn_block_pre_backward(*pre, H, K, V, d["dq"], d["dk"], d["dv"], d["db"], d["dg"], gate_is_log=True)

        cfg = {"workload": "gdn_block", **w, "io": "bf16", "what": "conv+SiLU+L2-norm/gate/beta and norm x gate, fwd+bwd"}
    elif args.workload == "mamba3_block":
        w = dict(WORKLOADS["mamba3_block"])
        if args.batch > 0:
            w["B"] = args.batch
        B, T, D, N, G, K = w["B"], w["T"], w["D"], w["N"], w["G"], w["K"]
        g = torch.Generator().manual_seed(5000 + rank)
        rn = lambda *shape: torch.randn(*shape, generator=g)
        io = torch.bfloat16
        d = dict(x=rn(B, T, D).to(io), cw=0.4 * rn(D, K), dyc=rn(B, T, D).to(io),
                 bp=rn(B, T, G * N).to(io), cp=rn(B, T, G * N).to(io), bs=1 + 0.2 * rn(N), cs=1 + 0.2 * rn(N),
                 bb=0.3 * rn(G * N), cb=0.3 * rn(G * N), db=rn(B, T, G, N).to(io), dc=rn(B, T, G, N).to(io),
                 y=rn(B, T, D).to(io), z=rn(B, T, D).to(io), pn=1 + 0.2 * rn(D), dout=rn(B, T, D).to(io))
        d = {k: v.to(dev) for k, v in d.items()}
        units = B * T
        metric, unit, dtype = "mamba3_block_stages_fwd_bwd_tokens_per_s", "tokens/s", "f32"
        alg_bytes = units * M3_BLOCK_BYTES_PER_TOKEN(D, G * N)
        alg_flops = 0.0
        bound = "hbm"
        traffic, traffic_note = None, "not captured"

        def step():
            ops.mamba3_block_conv(d["x"], d["cw"])
            ops.mamba3_block_bc(d["bp"], d["cp"], d["bs"], d["cs"], d["bb"], d["cb"], G, N)
            ops.mamba3_block_post(d["y"], d["z"], d["pn"])
            ops.mamba3_block_post_backward(d["y"], d["z"], d["pn"], d["dout"])
            ops.mamba3_block_bc_backward(d["bp"], d["cp"], d["bs"], d["cs"], d["db"], d["dc"], G, N)
            ops.mamba3_block_conv_backward(d["x"], d["cw"], d["dyc"])

        cfg = {"workload": "mamba3_block", **w, "io": "bf16", "what": "depthwise conv, B/C norm + bias, post-norm x gate, fwd+bwd"}
    else:
        w = dict(WORKLOADS["mamba3_train"])
        if args.batch > 0:
            w["B"] = args.batch
        B, T, NH, P, N, G = w["B"], w["T"], w["nheads"], w["headdim"], w["N"], w["G"]
        parts = [inputs.mamba3_inputs(1, T, NH, P, N, G=G, seed=3000 * (rank + 1) + b, io_dtype=torch.bfloat16)
                 for b in range(B)]
        keys = ("x", "dt_raw", "lambda_raw", "theta", "b", "c", "dy")
        d = {k: torch.cat([p[k] for p in parts]).to(dev) for k in keys}
        d["a_log"] = parts[0]["a_log"].to(dev)
        units = B * T
        metric, unit, dtype = "mamba3_fwd_bwd_tokens_per_s", "tokens/s", "bf16"
        alg_bytes = units * M3_BYTES_PER_TOKEN
        alg_flops = units * M3_FLOPS_PER_TOKEN
        bound = "hbm"
        traffic = B * NH * ((T + 63) // 64) * M3_NCU_TRAFFIC_PER_CHUNK if (P, N) == (64, 128) else None
        traffic_note = "one-pass ncu capture (dram bytes read + written) of a full-size step, per (batch, head, chunk) unit x units"
        margs = [d[k] for k in ("x", "dt_raw", "lambda_raw", "theta", "a_log", "b", "c")]

        def step():
            ops.mamba3_selective_scan(*margs, nheads=NH, save_for_backward=True)
            ops.mamba3_selective_scan_backward(*margs, d["dy"], nheads=NH, use_saved=True)

        cfg = {"workload": "mamba3_train", **w, "io": "bf16", "layout": "head-broadcast dt/lambda/theta/a_log"}

    # ---- warm-up, then the timed region --------------------------------------
    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.25)
    lib.mxb_trace_enable(1)
    n0 = lib.mxb_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.time()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    t_wall1 = time.time()
    ms = ev0.elapsed_time(ev1)
    launches = int(lib.mxb_launch_count() - n0)
    buf = C.create_string_buffer(1 << 16)
    lib.mxb_trace_summary(buf, len(buf))
    lib.mxb_trace_enable(0)
    clocks = sampler.stop(t_wall0, t_wall1)
    ms = sharding.max_over_ranks(ms, dev)
    kernels = {}
    for line in buf.value.decode().splitlines():
        name, cnt, tot = line.split()
        kernels[name] = dict(launches=int(cnt), total_ms=float(tot))
    ksum = sum(k["total_ms"] for k in kernels.values()) or 1.0
    for k in kernels.values():
        k["share"] = k["total_ms"] / ksum
        k["avg_ms"] = k["total_ms"] / max(k["launches"], 1)
    top = max(kernels, key=lambda n: kernels[n]["total_ms"]) if kernels else None

    ms_step = ms / args.steps
    value = sharding.whole_job_rate(units, world, ms_step * 1e-3)
    # roofline of the step, taken as one launch: algorithmic bytes / summed kernel time
    kern_ms_step = ksum / args.steps
    achieved = alg_bytes / (kern_ms_step * 1e-3) / 1e9
    roofline = {"bound": bound, "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                "frac": achieved / pk["hbm"], "traffic": traffic, "traffic_note": traffic_note, "peak_source": pk["src"],
                "scope": "all kernels of one step (algorithmic bytes of the step / summed kernel time)",
                "top_kernel": top, "kernels": kernels,
                "tensor_tflops": alg_flops / (kern_ms_step * 1e-3) / 1e12,
                "tensor_frac_of_sustained": alg_flops / (kern_ms_step * 1e-3) / 1e12 / pk["tf_sus"]}

    # ---- end to end through the host-buffer C ABI (gdn_train only) -----------
    if args.workload == "gdn_train" and not args.no_e2e:
        ctx = C.c_void_p()
        desc = mixlab_b200.GdnDesc(B, T, H, K, V, Cc, mixlab_b200.MXB_BF16, 1, flags)
        need = lib.mxb_gdn_bwd_workspace_bytes(C.byref(desc)) + 12 * B * T * H * max(K, V) * 2 + (64 << 20)
        del d
        torch.cuda.empty_cache()
        st = lib.mxb_host_ctx_create(local, need, C.byref(ctx))
        if st == 0:
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
            nst = max(2, min(args.steps, 5))
            barrier()
            t0 = time.perf_counter()
            for _ in range(nst):
                host_step()  # blocking: H2D + kernels + D2H + stream sync
            barrier()
            dt = (time.perf_counter() - t0) / nst
            dt = sharding.max_over_ranks(dt, dev)
            lib.mxb_host_ctx_destroy(ctx)
            h2d = sum(host[k].numel() * host[k].element_size() for k in ("q", "k", "v", "beta", "g", "d_out"))
            d2h = sum(t.numel() * t.element_size() for t in res.values())
            e2e = {"value": world * units / dt, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "ms_per_step": dt * 1e3, "api": "mxb_host_gdn (pinned host buffers, blocking)"}
        else:
            e2e = {"value": None, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                   "error": f"mxb_host_ctx_create status {st}"}

    cpu = None
    if rank == 0 and world == 1 and args.workload == "gdn_train" and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        tok, times = cpu_gdn_sample(threads, 2)
        cpu = {"value": tok / (sum(times) / len(times)), "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"B=1 of 8 sequences (T=4096, H=16, d=128), fp32, {len(times)} passes of "
                         "oracle.gdn.scan_chunked + torch autograd"}

    if rank == 0:
        print(json.dumps({
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": cfg,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
