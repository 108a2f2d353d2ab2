#!/usr/bin/env python
"""Benchmark of the GGUF quantized-weight linear layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--workload NAME] [--impl reference]

Default workload (N = 1): the Q4_0 decode GEMV pair at Llama-7B FFN shapes, batch 1 — one step
is y1 = W_up . x (K=4096 -> N=11008) followed by y2 = W_down . y1 (K=11008 -> N=4096), weights as
raw GGUF Q4_0 blocks, f32 activations, f32 outputs.  Metric: HBM GB/s = algorithmic bytes
(packed W + x + y of both launches, each counted once) / time.

Timing: CUDA events on the launching stream, W >= 3 warm-up steps, a barrier and a device
synchronise on both sides, max over ranks.  Successive steps use different weight copies (the
rotation set is larger than twice the 126 MB L2), so every step streams its weights from HBM.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    # name: (scheme name, [(k, n), ...] chained projections, activation dtype)
    "q4_0_llama7b_ffn_gemv": ("q4_0", [(4096, 11008), (11008, 4096)], "f32"),
    "q8_0_4096_gemv": ("q8_0", [(4096, 4096)], "f32"),
    "q4_k_8b_up_gemv": ("q4_k", [(4096, 14336)], "bf16"),
    "q6_k_8b_down_gemv": ("q6_k", [(14336, 4096)], "bf16"),
}
# Prefill GEMMs (configurations 4 and 2): name -> (scheme, m, k, n); bf16 activations and outputs.
GEMM_WORKLOADS = {
    "q8_0_prefill_gemm": ("q8_0", 4096, 8192, 28672),
    "q4_0_prefill_gemm": ("q4_0", 4096, 8192, 28672),
    "q4_k_8b_prefill_gemm": ("q4_k", 512, 4096, 14336),
}
# Tensor-parallel SwiGLU FFN at 70B shapes (configuration 3): handled by run_tp_workload.
TP_WORKLOAD = "q4_k_70b_ffn_tp"
# Tied LM head (greedy decode): name -> (scheme, n_embd, n_vocab); bf16 hidden state, exact re-ranking on.
LM_WORKLOADS = {
    "q4_k_lm_head_128k_argmax": ("q4_k", 4096, 128256),
    "q6_k_lm_head_128k_argmax": ("q6_k", 4096, 128256),
}
TP_D_MODEL, TP_D_FFN = 8192, 28672
SCHEME_IDS = {"q4_k": 0, "q6_k": 2, "q4_0": 6, "q8_0": 7}
GEOM = {"q4_k": (256, 144), "q6_k": (256, 210), "q4_0": (32, 18), "q8_0": (32, 34)}


def packed_bytes(sch: str, k: int, n: int) -> int:
    be, bb = GEOM[sch]
    return k * n // be * bb


def algorithmic_bytes(sch: str, layers, m: int, act_bytes: int) -> list[int]:
    """Per launch: packed W + x + y (f32 y), each once."""
    return [packed_bytes(sch, k, n) + m * k * act_bytes + m * n * 4 for k, n in layers]


def finish_ranks(dist, torch) -> None:
    """Ends a multi-rank run: all ranks meet, flush and leave.  Tearing the NCCL process group down
    while captured graphs that hold its kernels are alive has been seen to block for minutes (CUDA 12.9,
    NCCL 2.28), so the ranks exit directly once every rank has printed what it has to print."""
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def all_peaks() -> dict:
    """Roofline denominators: the measured copy bandwidth and cuBLAS bf16 rates in MEASURED_PEAKS.json
    beside this file when it exists, else fixed fallback figures (and the line says which)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm": float(d["hbm_gbs"]), "tf_burst": float(d["bf16_tflops"]),
                "tf_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured": True}
    return {"hbm": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "measured": False}


def measured_peaks() -> tuple[float, str]:
    pk = all_peaks()
    return pk["hbm"], ("measured (MEASURED_PEAKS.json hbm_gbs)" if pk["measured"]
                       else "fallback (6.65 TB/s, an earlier B200 copy measurement)")


def captured_traffic(workload: str, m: int):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu capture
    summary of this workload under profiles/ (a line `traffic: workload=<name> batch=<m> dram_bytes_per_launch=<N>`);
    None when no capture of this workload and batch is on file."""
    import glob
    import re
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        with open(path) as f:
            for ln in f:
                mt = re.search(r"traffic:\s*workload=(\S+)\s+batch=(\d+)\s+dram_bytes_per_launch=(\d+)", ln)
                if mt and mt.group(1) == workload and int(mt.group(2)) == m:
                    return int(mt.group(3))
    return None


def time_graph(torch, step, steps: int, warmup: int) -> float:
    """ms per step: `warmup` eager steps, then `steps` steps captured once in a CUDA graph, one untimed
    replay, one replay timed with CUDA events on the launching stream."""
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(steps):
            step(warmup + i)
    graph.replay()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    graph.replay()
    ev1.record()
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1) / steps


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()          # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------
# CPU baseline (the oracle = a port of the reference's CPU path; see oracle/rlxq_oracle.h)
# --------------------------------------------------------------------------------------------
def cpu_step(O, sch_id, layers, weights, x, threads):
    cur = x
    m = x.shape[0]
    for (k, n), w in zip(layers, weights):
        cur = O.matmul_bt_mt(cur, w, m, k, n, sch_id, threads=threads)
    return cur


def cpu_baseline(sch: str, layers, m: int, act: str, budget_s: float = 12.0) -> dict:
    from oracle import oracle as O
    sid = O.SCHEMES[sch]
    weights = [O.fill_weights(sid, 1000 + i, k, n) for i, (k, n) in enumerate(layers)]
    x = O.fill_normal(77, m * layers[0][0]).reshape(m, layers[0][0])
    cores = os.cpu_count() or 1
    total_bytes = sum(algorithmic_bytes(sch, layers, m, 4 if act == "f32" else 2))
    out = {}
    for label, threads in (("all_cores", cores), ("one_thread", 1)):
        cpu_step(O, sid, layers, weights, x, threads)            # warm
        t0 = time.perf_counter(); reps = 0
        while True:
            cpu_step(O, sid, layers, weights, x, threads); reps += 1
            if time.perf_counter() - t0 > budget_s / 2 or reps >= 20:
                break
        dt = (time.perf_counter() - t0) / reps
        out[label] = {"gbs": total_bytes / dt / 1e9, "ms_per_step": dt * 1e3, "threads": threads, "reps": reps}
    return {"value": out["all_cores"]["gbs"], "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{out['all_cores']['reps']} full steps of the same workload (all {cores} host threads, rows split "
                      f"across threads); single thread (what the reference runs): {out['one_thread']['gbs']:.3f} GB/s, "
                      f"{out['one_thread']['ms_per_step']:.1f} ms/step",
            "one_thread_value": out["one_thread"]["gbs"], "ms_per_step": out["all_cores"]["ms_per_step"]}


def run_reference_arm(args, rank: int, world: int) -> None:
    """The reference's CPU implementation of the path, timed on the host cores.  The reference is
    Rust and cannot be built in this image, so this is the oracle port of it."""
    if rank != 0:
        return
    sch, layers, act = WORKLOADS[args.workload]
    from oracle import oracle as O
    sid = O.SCHEMES[sch]
    m = args.batch
    # the same rotation of distinct weight copies as the GPU arm (same `config`), so no step finds its
    # weights in a cache; the copies are byte copies of one generated set
    w_step = sum(packed_bytes(sch, k, n) for k, n in layers)
    rotation = max(2, -(-2 * L2_BYTES // w_step) + 1)
    base = [O.fill_weights(sid, 1000 + i, k, n) for i, (k, n) in enumerate(layers)]
    wsets = [base] + [[w.copy() for w in base] for _ in range(rotation - 1)]
    x = O.fill_normal(77, m * layers[0][0]).reshape(m, layers[0][0])
    cores = os.cpu_count() or 1
    for i in range(args.warmup):
        cpu_step(O, sid, layers, wsets[i % rotation], x, cores)
    t0 = time.perf_counter()
    for i in range(args.steps):
        cpu_step(O, sid, layers, wsets[(args.warmup + i) % rotation], x, cores)
    dt = (time.perf_counter() - t0) / args.steps
    total_bytes = sum(algorithmic_bytes(sch, layers, m, 4 if act == "f32" else 2))
    val = total_bytes / dt / 1e9
    line = {
        "impl": "reference", "metric": "gemv_hbm_gbs", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, sch, layers, act, rotation),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} full steps, all {cores} host threads (rows split across threads)"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, sch, layers, act, rotation):
    return {"workload": args.workload, "scheme": sch, "batch": args.batch, "gemv_kernel": getattr(args, "gemv_kernel", 0),
            "layers_k_to_n": [[k, n] for k, n in layers], "activations": act, "output": "f32",
            "l2": f"rotating {rotation} distinct weight copies per rank "
                  f"({rotation * sum(packed_bytes(sch, k, n) for k, n in layers) / 1e6:.0f} MB) > 2 x 126 MB L2"}




# --------------------------------------------------------------------------------------------
# Prefill GEMM (configurations 4 and 2): compute-bound, TFLOP/s against the dense bf16 peak
# --------------------------------------------------------------------------------------------
def run_gemm_workload(args, rank, world, local_rank):
    sch, m, k, n = GEMM_WORKLOADS[args.workload]
    if args.gemm_shape:
        m, k, n = (int(v) for v in args.gemm_shape.split(","))
    flops = 2.0 * m * k * n
    cfg = {"workload": args.workload, "scheme": sch, "m": m, "k": k, "n": n, "activations": "bf16", "output": "bf16",
           "l2": "operands larger than L2: packed W %.0f MB + x %.0f MB + y %.0f MB" %
                 (packed_bytes(sch, k, n) / 1e6, m * k * 2 / 1e6, m * n * 2 / 1e6)}
    from oracle import oracle as O
    sid = O.SCHEMES[sch]
    if args.impl == "reference":
        if rank != 0:
            return
        # bounded sample of the same workload: 64 token rows x 128 weight rows x all of k, scaled by work
        cores = os.cpu_count() or 1
        rb = packed_bytes(sch, k, 1)
        w = O.fill_weights(sid, 3000, k, 128)
        x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(79, 64 * k))).reshape(64, k)
        O.matmul_bt_mt(x, w, 64, k, 128, sid, threads=cores)
        steps = min(args.steps, 10)
        t0 = time.perf_counter()
        for _ in range(steps):
            O.matmul_bt_mt(x, w, 64, k, 128, sid, threads=cores)
        dt = (time.perf_counter() - t0) / steps
        val = 2.0 * 64 * k * 128 / dt / 1e12
        print(json.dumps({"impl": "reference", "metric": "gemm_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
                          "steps": steps, "warmup": args.warmup, "ms_per_step": flops / (val * 1e12) * 1e3,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": cfg,
                          "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                           "sample": f"64 token rows x 128 weight rows x k={k} per step ({rb * 128} weight bytes), "
                                                     f"all {cores} host threads; ms_per_step is scaled to the full shape"},
                          "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rlxq kernels have no CPU path")
    import rlx_b200 as R
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w_host = O.fill_weights(sid, 3000 + rank, k, n)
    wd = torch.from_numpy(w_host).to(dev)
    x_host = O.fill_normal(79 + rank, m * k).reshape(m, k)
    xd = torch.from_numpy(x_host).to(dev).to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        R.matmul(xd, wd, SCHEME_IDS[sch], n, out=y)
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = R.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    ev0.record()
    for _ in range(args.steps):
        R.matmul(xd, wd, SCHEME_IDS[sch], n, out=y)
    ev1.record()
    sync_all()
    R.device_status()
    launches = R.launch_count() - launches0
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    # end to end: Graph / Session API, x and y in pinned host memory as raw bf16 bytes
    g = R.Graph("gemm")
    xi = g.input("x", [m, k], R.DType.BF16)
    p = g.param("w", [len(w_host)])
    g.set_outputs([g.dequant_matmul_packed(xi, p, R.QuantScheme(SCHEME_IDS[sch]), n, R.DType.BF16)])
    c = R.Session(R.Device.Cuda, index=local_rank, exec_mode="graph").compile(g)
    c.set_param_typed("w", w_host, R.DType.U8)
    x_pin = xd.cpu().pin_memory()
    y_pin = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(2, min(args.steps, 10))
    for _ in range(2):
        c.run_raw(["x"], [x_pin.data_ptr()], [m * k * 2], [1], y_pin.data_ptr(), m * n * 2, 1)
    sync_all()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        c.run_raw(["x"], [x_pin.data_ptr()], [m * k * 2], [1], y_pin.data_ptr(), m * n * 2, 1)
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    torch.cuda.synchronize()
    e2e_ok = bool(torch.equal(y_pin, y.cpu()))
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    if rank == 0:
        peaks = {}
        pth = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(pth):
            with open(pth) as f:
                peaks = json.load(f)
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0)) if ms > 100.0 else float(peaks.get("bf16_tflops", 1590.0))
        src = ("measured (MEASURED_PEAKS.json, %s)" % ("sustained: the timed region is a long back-to-back loop" if ms > 100.0 else "burst")
               if peaks else "fallback (1.59 PFLOP/s burst / 1.4 sustained, earlier measurement on this pool)")
        ach = flops / (ms_per_step * 1e-3) / 1e12
        line = {"metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg, "clocks": clocks,
                "e2e": {"value": world * flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": m * k * 2,
                        "d2h_bytes_per_step": m * n * 2, "ms_per_step": e2e_s * 1e3, "matches_resident_path": e2e_ok,
                        "api": "Session(Device.Cuda).compile(graph).run_typed, pinned host buffers"},
                "gpu_launches": launches,
                "roofline": {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                             "peak_source": src, "frac_of_burst": ach / float(peaks.get("bf16_tflops", 1590.0)),
                             "frac_of_nominal_2250": ach / 2250.0,
                             "kernel": "gemm_pair_kernel (two CTAs per MMA)" if R.get_option("gemm_pair_clusters") > 0 else "gemm_tcgen05_kernel",
                             "flops_per_launch": flops, "avg_launch_us": ms_per_step * 1e3,
                             "traffic": packed_bytes(sch, k, n) + m * k * 2 + m * n * 2}}
        if not args.no_cpu_baseline and world == 1:
            cores = os.cpu_count() or 1
            wsub = O.fill_weights(sid, 3000, k, 128)
            xs = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(79, 64 * k))).reshape(64, k)
            O.matmul_bt_mt(xs, wsub, 64, k, 128, sid, threads=cores)
            t0 = time.perf_counter(); reps = 0
            while time.perf_counter() - t0 < 8.0 and reps < 20:
                O.matmul_bt_mt(xs, wsub, 64, k, 128, sid, threads=cores); reps += 1
            dt = (time.perf_counter() - t0) / reps
            line["cpu_baseline"] = {"value": 2.0 * 64 * k * 128 / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"{reps} passes over 64 token rows x 128 weight rows x k={k}, all {cores} host threads"}
        print(json.dumps(line), flush=True)
    if world > 1:
        finish_ranks(dist, torch)

# --------------------------------------------------------------------------------------------
# Tensor-parallel FFN (configuration 3): strong scaling, one NCCL all-reduce per step
# --------------------------------------------------------------------------------------------
def tp_bytes(m: int) -> int:
    """Algorithmic bytes of one FFN pass: three packed Q4_K projections + bf16 x + f32 y."""
    return 3 * packed_bytes("q4_k", TP_D_MODEL, TP_D_FFN) + m * TP_D_MODEL * 2 + m * TP_D_MODEL * 4


def tp_flops(m: int) -> float:
    """Multiply-adds x 2 of one FFN pass: three projections of d_model x d_ffn."""
    return 2.0 * m * 3 * TP_D_MODEL * TP_D_FFN


def tp_config(args, world, rotation, reduce_kind="nccl"):
    return {"all_reduce": reduce_kind if world > 1 else "none", "tp_fused": int(args.tp_fused), "workload": TP_WORKLOAD, "scheme": "q4_k", "batch": args.batch, "d_model": TP_D_MODEL, "d_ffn": TP_D_FFN,
            "parallelism": f"tp{world}: gate/up column-split, down row-split, all-reduce of f32 partials",
            "activations": "bf16", "output": "f32",
            "l2": f"rotating {rotation} distinct shard sets per rank > 2 x 126 MB L2"}


def run_tp_reference_arm(args, rank, world):
    """The reference's CPU path for configuration 3 (the oracle port of it), all host threads.  A decode batch
    runs whole FFN passes; a prefill batch runs a bounded sample of 8 of its token rows (rows are independent)
    and ms_per_step is scaled to the full batch."""
    if rank != 0:
        return
    from oracle import oracle as O
    m, dm, df = args.batch, TP_D_MODEL, TP_D_FFN
    gate, up, down = (O.fill_weights(O.Q4_K, 2000 + i, *sh) for i, sh in enumerate(((dm, df), (dm, df), (df, dm))))
    rows = min(m, 8)
    x = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(78, rows * dm))).reshape(rows, dm)
    cores = os.cpu_count() or 1
    steps = min(args.steps, 20)          # a bounded sample: one pass is ~0.7 G multiply-adds per token
    for _ in range(min(args.warmup, 3)):
        O.ffn_swiglu(x, gate, up, down, rows, dm, df, O.Q4_K, O.Q4_K, threads=cores)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.ffn_swiglu(x, gate, up, down, rows, dm, df, O.Q4_K, O.Q4_K, threads=cores)
    dt = (time.perf_counter() - t0) / steps
    if m <= 8:
        val, unit, metric, ms = tp_bytes(m) / dt / 1e9, "GB/s", "gemv_hbm_gbs", dt * 1e3
        sample = f"{steps} full FFN passes on all {cores} host threads"
    else:
        val, unit, metric, ms = tp_flops(rows) / dt / 1e12, "TFLOP/s", "gemm_tflops", dt * 1e3 * m / rows
        sample = f"{steps} FFN passes over {rows} of the {m} token rows on all {cores} host threads; ms_per_step scaled to {m} rows"
    g = max(1, args.gpus)
    shard = 3 * packed_bytes("q4_k", dm, df) // g
    rotation = max(2, -(-2 * L2_BYTES // shard) + 1)
    cfg = tp_config(args, g, rotation, "rank-order sum on the host" if g > 1 else "none")
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)


def run_tp_workload(args, rank, world, local_rank):
    """Configuration 3 on `world` GPUs.  The headline is the batch given by --batch (1 unless stated): HBM GB/s
    for a decode batch, TFLOP/s for a prefill batch; unless --no-sweep is given the other batch of the
    configuration (256 / 1) follows as a `configs` entry.  Rank 0 checks its summed result against the oracle FFN."""
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rlxq kernels have no CPU path")
    import rlx_b200 as R
    from rlx_b200 import tp
    from oracle import oracle as O
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    R.set_option("tp_fused", args.tp_fused)
    dm, df = TP_D_MODEL, TP_D_FFN
    plan = tp.shard_plan(O.Q4_K, dm, df, world, rank)
    shard_bytes = 2 * plan.gate_up_bytes + plan.down_bytes
    rotation = max(2, -(-2 * L2_BYTES // shard_bytes) + 1)
    # every rank generates only its own shards: blocks are counter-based, so a shard of the seeded
    # full tensor is a sub-range of its block stream (gate/up) or a strided set of sub-ranges (down)
    be = 256
    ffns = []
    for r in range(rotation):
        seeds = [2000 + 10 * r + i for i in range(3)]
        first = plan.ffn_begin * (dm // be)
        gu = np.concatenate([O.fill_blocks(O.Q4_K, seeds[0], plan.ffn_local * dm // be, first),
                             O.fill_blocks(O.Q4_K, seeds[1], plan.ffn_local * dm // be, first)])
        per_row, loc = df // be, plan.ffn_local // be
        dn = np.concatenate([O.fill_blocks(O.Q4_K, seeds[2], loc, j * per_row + plan.ffn_begin // be) for j in range(dm)])
        f = tp.TensorParallelFFN(O.Q4_K, dm, df, rank=rank, world=world, device=dev)
        f.load_shards(gu, dn)
        ffns.append(f)
    # decode-sized partials are summed by the one-shot peer-memory all-reduce; larger ones, or when the peer
    # mapping cannot be set up (or RLXQ_TP_ALLREDUCE=nccl), by the process group's
    pr = None
    if world > 1 and os.environ.get("RLXQ_TP_ALLREDUCE", "peer") == "peer":
        pr = tp.PeerAllReduce(rank, world)
        if pr.available:
            for f in ffns:
                f.peer_reduce = pr
    full = None      # rank 0: the whole tensors of rotation set 0, for the oracle check

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def measure(m: int, steps: int, warmup: int, want_e2e: bool) -> dict:
        nonlocal full
        x_host = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(78, m * dm))).reshape(m, dm)
        x_dev = torch.from_numpy(x_host).to(dev).to(torch.bfloat16)
        y = torch.empty((m, dm), dtype=torch.float32, device=dev)
        reduce_kind = "none" if world == 1 else ("peer memory, one shot, rank order" if pr is not None and pr.fits(y) else "nccl")

        def step(i):
            ffns[i % rotation].forward(x_dev, out=y)

        for i in range(warmup):
            step(i)
        sync_all()
        launches0 = R.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(steps):
                step(warmup + i)
        launches = R.launch_count() - launches0
        graph.replay()
        sync_all()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        ev0.record()
        graph.replay()
        ev1.record()
        sync_all()
        R.device_status()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            tt = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
            lt = torch.tensor([launches], dtype=torch.int64, device=dev)
            dist.all_reduce(lt, op=dist.ReduceOp.SUM)
            launches = int(lt.item())
        clocks = sampler.stop() if rank == 0 else None
        res = {"m": m, "ms_per_step": ms / steps, "steps": steps, "launches": launches, "clocks": clocks,
               "reduce_kind": reduce_kind, "parity_max": None}
        # rank 0: the summed result of rotation set 0 against the oracle FFN on sampled token rows
        step(0)
        sync_all()
        if rank == 0:
            if full is None:
                full = tuple(O.fill_weights(O.Q4_K, 2000 + i, *sh) for i, sh in enumerate(((dm, df), (dm, df), (df, dm))))
            rows = np.arange(m) if m <= 8 else np.unique(np.linspace(0, m - 1, 4).astype(np.int64))
            res["parity_max"] = tp_oracle_check(O, x_host, y.cpu().numpy(), *full, dm, df, rows)
            res["parity_sample"] = "every output" if m <= 8 else f"{len(rows)} token rows, every output"
        if want_e2e:
            # end to end: x from pinned host memory every step, y back to pinned host memory
            x_pin = torch.from_numpy(x_host).to(torch.bfloat16).pin_memory()
            y_pin = torch.empty((m, dm), dtype=torch.float32).pin_memory()

            def e2e_step(i):
                x_dev.copy_(x_pin, non_blocking=True)
                ffns[i % rotation].forward(x_dev, out=y)
                y_pin.copy_(y, non_blocking=True)
                torch.cuda.synchronize()

            for i in range(warmup):
                e2e_step(i)
            sync_all()
            t0 = time.perf_counter()
            for i in range(steps):
                e2e_step(warmup + i)
            e2e_s = time.perf_counter() - t0
            if world > 1:
                tt = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                e2e_s = float(tt.item())
            res["e2e_s_per_step"] = e2e_s / steps
        return res

    def rate(m: int, s_per_step: float) -> tuple[float, str, str]:
        if m <= 8:
            return tp_bytes(m) / s_per_step / 1e9, "GB/s", "gemv_hbm_gbs"
        return tp_flops(m) / s_per_step / 1e12, "TFLOP/s", "gemm_tflops"

    def roofline_of(m: int, ms_per_step: float, pk: dict) -> dict:
        if m <= 8:
            per_gpu = (shard_bytes + m * dm * 6) / (ms_per_step * 1e-3) / 1e9
            return {"bound": "hbm", "achieved": per_gpu, "peak": pk["hbm"], "unit": "GB/s", "frac": per_gpu / pk["hbm"],
                    "peak_source": "measured copy bandwidth (MEASURED_PEAKS.json)" if pk["measured"] else "fallback 6.65 TB/s",
                    "frac_of_nominal_8TBs": per_gpu / 8000.0,
                    "kernel": "the GEMV kernels of one FFN step (per GPU: its shard bytes / whole step time, all-reduce included)",
                    "bytes_per_step_per_gpu": shard_bytes + m * dm * 6, "traffic": None}
        per_gpu = tp_flops(m) / world / (ms_per_step * 1e-3) / 1e12
        return {"bound": "tensor", "achieved": per_gpu, "peak": pk["tf_burst"], "unit": "TFLOP/s", "frac": per_gpu / pk["tf_burst"],
                "peak_source": "measured cuBLAS bf16 burst (MEASURED_PEAKS.json)" if pk["measured"] else "fallback 1.59 PFLOP/s",
                "frac_of_sustained": per_gpu / pk["tf_sustained"],
                "kernel": "gemm_tcgen05_kernel x 2 + the SwiGLU kernel (per GPU: its share of the FLOPs / whole step time, all-reduce included)",
                "flops_per_step_per_gpu": tp_flops(m) / world, "traffic": None}

    m = args.batch
    head = measure(m, args.steps if m <= 8 else min(args.steps, 20), args.warmup, True)
    other = None
    if not args.no_sweep and m in (1, 256):
        om = 256 if m == 1 else 1
        other = measure(om, 20 if om > 8 else 100, 3, False)
    if rank == 0:
        pk = all_peaks()
        value, unit, metric = rate(m, head["ms_per_step"] * 1e-3)
        e2e_val = rate(m, head["e2e_s_per_step"])[0]
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": head["steps"],
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32" if m <= 8 else "bf16", "data": "synthetic",
            "config": tp_config(args, world, rotation, head["reduce_kind"]),
            "clocks": head["clocks"],
            "e2e": {"value": e2e_val, "unit": unit, "h2d_bytes_per_step": m * dm * 2, "d2h_bytes_per_step": m * dm * 4,
                    "ms_per_step": head["e2e_s_per_step"] * 1e3,
                    "api": "TensorParallelFFN.forward: pinned x -> device, rlxq_tp_ffn_step (partial + all-reduce), y -> pinned host"},
            "gpu_launches": head["launches"],
            "roofline": roofline_of(m, head["ms_per_step"], pk),
            "parity_max": head["parity_max"], "parity_sample": head.get("parity_sample"),
        }
        if other is not None:
            ov, ou, om_metric = rate(other["m"], other["ms_per_step"] * 1e-3)
            line["configs"] = [{"name": f"cfg3 q4_k 70b ffn m={other['m']}, {world} gpu", "m": other["m"], "metric": om_metric,
                                "value": ov, "unit": ou, "ms": other["ms_per_step"], "all_reduce": other["reduce_kind"],
                                "roofline": roofline_of(other["m"], other["ms_per_step"], pk),
                                "parity_max": other["parity_max"], "parity_sample": other.get("parity_sample")}]
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            gate, up, down = full
            ms_rows = min(m, 8)                 # a bounded sample for a prefill batch: 8 of its token rows
            xx = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(78, ms_rows * dm))).reshape(ms_rows, dm)
            O.ffn_swiglu(xx, gate, up, down, ms_rows, dm, df, O.Q4_K, O.Q4_K, threads=cores)
            t0 = time.perf_counter(); reps = 0
            while time.perf_counter() - t0 < 8.0 and reps < 20:
                O.ffn_swiglu(xx, gate, up, down, ms_rows, dm, df, O.Q4_K, O.Q4_K, threads=cores); reps += 1
            dt = (time.perf_counter() - t0) / reps
            line["cpu_baseline"] = {"value": rate(ms_rows, dt)[0] if m <= 8 else tp_flops(ms_rows) / dt / 1e12, "unit": unit,
                                    "cores": cores, "kind": "port",
                                    "sample": f"{reps} FFN passes over {ms_rows} token rows, all {cores} host threads",
                                    "ms_per_step": dt * 1e3}
        print(json.dumps(line), flush=True)
    if world > 1:
        finish_ranks(dist, torch)

# --------------------------------------------------------------------------------------------
# Every configuration on one line: the default run appends a `configs` list to the headline, each entry
# measured the same way (resident inputs, CUDA graph, CUDA events, weights rotated past L2 or larger than
# it) and checked against an oracle sample taken in the same run.
# --------------------------------------------------------------------------------------------
def parity_ratio(y, ref, xn, wn) -> float:
    """worst |y - y_ref| / (||x_row|| ||w_row||) over the sample."""
    err = np.abs(np.asarray(y, np.float64) - np.asarray(ref, np.float64))
    return float((err / np.maximum(xn[:, None] * wn[None, :], 1e-30)).max())


def sweep_gemv(torch, R, O, dev, name, sch, layers, act, m, steps, warmup, pk) -> dict:
    sid = O.SCHEMES[sch]
    act_t = torch.float32 if act == "f32" else torch.bfloat16
    w_host = [O.fill_weights(sid, 5000 + i, k, n) for i, (k, n) in enumerate(layers)]
    w_step = sum(w.size for w in w_host)
    rotation = max(2, -(-2 * L2_BYTES // w_step) + 1)
    base = [torch.from_numpy(w).to(dev) for w in w_host]
    wsets = [base] + [[b.clone() for b in base] for _ in range(rotation - 1)]    # same bytes at other addresses
    x_host = O.fill_normal(81, m * layers[0][0]).reshape(m, layers[0][0])
    if act != "f32":
        x_host = O.bf16_bits_to_f32(O.f32_to_bf16_bits(x_host)).reshape(m, -1)
    x_dev = torch.from_numpy(x_host).to(dev).to(act_t)
    outs = [torch.empty((m, n), dtype=torch.float32, device=dev) for _, n in layers]
    need = max(R.workspace_bytes(sid, m, k, n, 0 if act == "f32" or i else 1, 0) for i, (k, n) in enumerate(layers))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)

    def step(i):
        cur = x_dev
        for li, (_, n) in enumerate(layers):
            R.matmul(cur, wsets[i % rotation][li], sid, n, out=outs[li], workspace=ws)
            cur = outs[li]

    l0 = R.launch_count()
    step(0)
    per_step_launches = R.launch_count() - l0
    ms = time_graph(torch, step, steps, warmup)
    R.device_status()
    step(0)
    torch.cuda.synchronize()
    worst, cur = 0.0, x_host
    for li, (k, n) in enumerate(layers):            # every layer against the oracle on the input it really had
        y = outs[li].cpu().numpy()
        ref = O.matmul_bt_mt(cur, w_host[li], m, k, n, sid)
        xn = np.sqrt((cur.astype(np.float64) ** 2).sum(axis=1))
        worst = max(worst, parity_ratio(y, ref, xn, O.row_norms(sid, w_host[li], k, n)))
        cur = y
    by = sum(algorithmic_bytes(sch, layers, m, 4 if act == "f32" else 2))
    ach = by / (ms * 1e-3) / 1e9
    return {"name": name, "scheme": sch, "m": m, "layers_k_to_n": [[k, n] for k, n in layers], "activations": act,
            "metric": "gemv_hbm_gbs", "value": ach, "unit": "GB/s", "ms": ms, "launches_per_step": per_step_launches,
            "roofline": {"bound": "hbm", "frac": ach / pk["hbm"], "peak": pk["hbm"],
                         "peak_kind": "measured copy bandwidth" if pk["measured"] else "fallback"},
            "parity_max": worst, "parity_sample": "every output of every layer",
            "l2": f"{rotation} weight copies in rotation"}


def sweep_gemm(torch, R, O, dev, name, sch, m, k, n, steps, warmup, pk) -> dict:
    sid = O.SCHEMES[sch]
    w_host = O.fill_weights(sid, 5100, k, n)
    wd = torch.from_numpy(w_host).to(dev)
    x_host = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(82, m * k))).reshape(m, k)
    xd = torch.from_numpy(x_host).to(dev).to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    need = R.workspace_bytes(sid, m, k, n, 1, 1)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    small = packed_bytes(sch, k, n) + m * k * 2 + m * n * 2 < 2 * L2_BYTES
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev) if small else None

    def step(i):
        R.matmul(xd, wd, sid, n, out=y, workspace=ws)

    if small:
        # operands smaller than L2: time single launches, L2 flushed by a 252 MB fill in between
        for i in range(warmup):
            step(i)
        torch.cuda.synchronize()
        times = []
        for i in range(steps):
            flush.fill_(i & 0xFF)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(); step(i); ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1))
        ms = statistics.median(times)
    else:
        ms = time_graph(torch, step, steps, warmup)
    R.device_status()
    # oracle sample: 16 token rows spread over m against two slabs of 64 weight rows
    rows = np.unique(np.linspace(0, m - 1, 16).astype(np.int64))
    rb = packed_bytes(sch, k, 1)
    worst = 0.0
    yh = y.float().cpu().numpy()
    xs = np.ascontiguousarray(x_host[rows])
    xn = np.sqrt((xs.astype(np.float64) ** 2).sum(axis=1))
    for r0 in (0, max(0, (n // 2) // 64 * 64), max(0, n - 64)):
        r1 = min(n, r0 + 64)
        wsub = w_host[r0 * rb:r1 * rb]
        ref = O.matmul_bt_mt(xs, wsub, len(rows), k, r1 - r0, sid)
        worst = max(worst, parity_ratio(yh[rows][:, r0:r1], ref, xn, O.row_norms(sid, wsub, k, r1 - r0)))
    flops = 2.0 * m * k * n
    ach = flops / (ms * 1e-3) / 1e12
    return {"name": name, "scheme": sch, "m": m, "k": k, "n": n, "activations": "bf16", "output": "bf16",
            "metric": "gemm_tflops", "value": ach, "unit": "TFLOP/s", "ms": ms,
            "roofline": {"bound": "tensor", "frac": ach / pk["tf_burst"], "peak": pk["tf_burst"],
                         "peak_kind": "measured cuBLAS bf16 burst" if pk["measured"] else "fallback",
                         "frac_of_sustained": ach / pk["tf_sustained"]},
            "parity_max": worst, "parity_sample": f"{len(rows)} token rows x 3 slabs of 64 weight rows",
            "l2": "L2 flushed between single timed launches" if small else "operands larger than L2"}


def tp_oracle_check(O, x_host_bf16_as_f32, y, gate, up, down, dm, df, rows) -> float:
    """Rank 0's FFN result against the oracle FFN on the sampled token rows (rows are independent)."""
    xs = np.ascontiguousarray(x_host_bf16_as_f32[rows])
    ref, h = O.ffn_swiglu(xs, gate, up, down, len(rows), dm, df, O.Q4_K, O.Q4_K, want_h=True)
    hn = np.sqrt((h.astype(np.float64) ** 2).sum(axis=1))
    return parity_ratio(y[rows], ref, hn, O.row_norms(O.Q4_K, down, df, dm))


def sweep_ffn_one_gpu(torch, R, O, dev, name, m, steps, warmup, pk) -> dict:
    from rlx_b200 import tp
    dm, df = TP_D_MODEL, TP_D_FFN
    gate, up, down = (O.fill_weights(O.Q4_K, 2000 + i, *sh) for i, sh in enumerate(((dm, df), (dm, df), (df, dm))))
    ffns = []
    for r in range(2):                               # 2 x 396 MB > 2 x L2
        f = tp.TensorParallelFFN(O.Q4_K, dm, df, rank=0, world=1, device=dev)
        if r == 0:
            f.load(gate, up, down)
        else:
            f.gate_up, f.down = ffns[0].gate_up.clone(), ffns[0].down.clone()
        ffns.append(f)
    x_host = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(78, m * dm))).reshape(m, dm)
    x_dev = torch.from_numpy(x_host).to(dev).to(torch.bfloat16)
    y = torch.empty((m, dm), dtype=torch.float32, device=dev)

    def step(i):
        ffns[i % 2].forward(x_dev, out=y)

    l0 = R.launch_count()
    step(0)
    per_step_launches = R.launch_count() - l0
    ms = time_graph(torch, step, steps, warmup)
    R.device_status()
    step(0)
    torch.cuda.synchronize()
    rows = np.arange(m) if m <= 8 else np.unique(np.linspace(0, m - 1, 4).astype(np.int64))
    worst = tp_oracle_check(O, x_host, y.cpu().numpy(), gate, up, down, dm, df, rows)
    out = {"name": name, "scheme": "q4_k", "m": m, "d_model": dm, "d_ffn": df, "activations": "bf16", "output": "f32",
           "ms": ms, "launches_per_step": per_step_launches, "parity_max": worst,
           "parity_sample": "every output" if m <= 8 else f"{len(rows)} token rows, every output",
           "l2": "2 weight sets of 396 MB in rotation"}
    if m <= 8:
        ach = tp_bytes(m) / (ms * 1e-3) / 1e9
        out.update({"metric": "gemv_hbm_gbs", "value": ach, "unit": "GB/s",
                    "roofline": {"bound": "hbm", "frac": ach / pk["hbm"], "peak": pk["hbm"],
                                 "peak_kind": "measured copy bandwidth" if pk["measured"] else "fallback"}})
    else:
        ach = tp_flops(m) / (ms * 1e-3) / 1e12
        out.update({"metric": "gemm_tflops", "value": ach, "unit": "TFLOP/s",
                    "roofline": {"bound": "tensor", "frac": ach / pk["tf_burst"], "peak": pk["tf_burst"],
                                 "peak_kind": "measured cuBLAS bf16 burst" if pk["measured"] else "fallback",
                                 "frac_of_sustained": ach / pk["tf_sustained"]}})
    return out


def sweep_all_configs(torch, R, O, dev, headline_entry: dict) -> list[dict]:
    """The configurations beside the headline one, one entry each; a failure becomes an entry with `error`."""
    pk = all_peaks()
    jobs = [
        lambda: sweep_gemv(torch, R, O, dev, "cfg0 q8_0 4096x4096 gemv m=1", "q8_0", [(4096, 4096)], "f32", 1, 200, 5, pk),
        lambda: sweep_gemv(torch, R, O, dev, "cfg1 q4_0 llama7b ffn gemv pair m=4", "q4_0", [(4096, 11008), (11008, 4096)], "f32", 4, 100, 5, pk),
        lambda: sweep_gemv(torch, R, O, dev, "cfg1 q4_0 llama7b ffn gemv pair m=8", "q4_0", [(4096, 11008), (11008, 4096)], "f32", 8, 100, 5, pk),
        lambda: sweep_gemv(torch, R, O, dev, "cfg2 q4_k 4096->14336 gemv m=1", "q4_k", [(4096, 14336)], "bf16", 1, 200, 5, pk),
        lambda: sweep_gemv(torch, R, O, dev, "cfg2 q6_k 14336->4096 gemv m=1", "q6_k", [(14336, 4096)], "bf16", 1, 200, 5, pk),
        lambda: sweep_gemv(torch, R, O, dev, "cfg2 q4_k 4096->14336 gemv m=4", "q4_k", [(4096, 14336)], "bf16", 4, 100, 5, pk),
        lambda: sweep_gemv(torch, R, O, dev, "cfg2 q4_k 4096->14336 gemv m=8", "q4_k", [(4096, 14336)], "bf16", 8, 100, 5, pk),
        lambda: sweep_gemv(torch, R, O, dev, "cfg2 q6_k 14336->4096 gemv m=4", "q6_k", [(14336, 4096)], "bf16", 4, 100, 5, pk),
        lambda: sweep_gemv(torch, R, O, dev, "cfg2 q6_k 14336->4096 gemv m=8", "q6_k", [(14336, 4096)], "bf16", 8, 100, 5, pk),
        lambda: sweep_gemm(torch, R, O, dev, "cfg2 q4_k 4096->14336 gemm m=512", "q4_k", 512, 4096, 14336, 20, 3, pk),
        lambda: sweep_gemm(torch, R, O, dev, "cfg2 q6_k 14336->4096 gemm m=512", "q6_k", 512, 14336, 4096, 20, 3, pk),
        lambda: sweep_ffn_one_gpu(torch, R, O, dev, "cfg3 q4_k 70b ffn m=1, 1 gpu", 1, 50, 3, pk),
        lambda: sweep_ffn_one_gpu(torch, R, O, dev, "cfg3 q4_k 70b ffn m=256, 1 gpu", 256, 10, 3, pk),
        lambda: sweep_gemm(torch, R, O, dev, "cfg4 q8_0 8192->28672 gemm m=4096", "q8_0", 4096, 8192, 28672, 5, 3, pk),
        lambda: sweep_gemm(torch, R, O, dev, "cfg4 q4_0 8192->28672 gemm m=4096", "q4_0", 4096, 8192, 28672, 5, 3, pk),
    ]
    out = [headline_entry]
    for job in jobs:
        try:
            out.append(job())
        except Exception as e:                      # one broken configuration must not hide the others
            out.append({"error": f"{type(e).__name__}: {e}"})
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
# MoE decode: name -> (scheme, k, n, experts, rows routed per step); f32 activations.
MOE_WORKLOADS = {
    "q4_k_moe_8x_top2_decode": ("q4_k", 4096, 14336, 8, 2),
    "q4_k_moe_64x_top8_decode": ("q4_k", 2048, 1408, 64, 8),
    # prefill-sized: 512 tokens x top-2 = 1024 rows over 8 experts (the grouped tensor-core GEMM)
    "q4_k_moe_8x_top2_prefill": ("q4_k", 4096, 14336, 8, 1024),
}


def run_moe_workload(args, rank, world, local_rank):
    """Op::DequantGroupedMatMul: `rows` token rows routed over the experts (decode sizes: each row to a different
    expert, GB/s over the routed slabs; prefill sizes: TFLOP/s)."""
    import torch
    if world != 1:
        raise SystemExit("the MoE workload is single-GPU")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rlxq kernels have no CPU path")
    import rlx_b200 as R
    from oracle import oracle as O      # input generation and the cpu_baseline leg only
    import numpy as np
    sch, k, n, E, rows = MOE_WORKLOADS[args.workload]
    sid = SCHEME_IDS[sch]
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    slab = packed_bytes(sch, k, n)
    prefill = rows > 8
    # decode: the routed experts only (the others are never read); prefill: every expert once
    step_bytes = (E * slab + rows * (k * 4 + n * 4)) if prefill else rows * (slab + k * 4 + n * 4)
    step_flops = 2.0 * rows * k * n
    rotation = max(2, -(-2 * L2_BYTES // (E * slab)) + 1)
    w_host = O.fill_weights(sid, 777, k, n * E)
    stacks = [torch.from_numpy(w_host).to(dev)] + [torch.from_numpy(O.fill_weights(sid, 778 + r, k, n * E)).to(dev)
                                                    for r in range(rotation - 1)]
    x_host = O.fill_normal(5, rows * k).reshape(rows, k)
    x_dev = torch.from_numpy(x_host).to(dev)
    routes = [torch.from_numpy(np.array([(7 * s + 3 * r) % E for r in range(rows)], np.float32)).to(dev) for s in range(8)]
    y = torch.empty((rows, n), dtype=torch.float32, device=dev)
    import ctypes as C
    from rlx_b200._lib import lib
    need = C.c_size_t()
    assert lib.rlxq_grouped_workspace_bytes(sid, rows, k, n, E, C.byref(need)) == 0
    wsb = torch.empty(max(need.value, 1 << 22), dtype=torch.uint8, device=dev)

    def step(i):
        R.grouped_matmul(x_dev, stacks[i % rotation], routes[i % 8], sid, n, E, out=y, workspace=wsb)

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    launches0 = R.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            step(args.warmup + i)
    launches = R.launch_count() - launches0
    graph.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ev0.record(); graph.replay(); ev1.record()
    torch.cuda.synchronize()
    R.device_status()
    clocks = sampler.stop()
    ms_per_step = ev0.elapsed_time(ev1) / args.steps
    value = step_flops / (ms_per_step * 1e-3) / 1e12 if prefill else step_bytes / (ms_per_step * 1e-3) / 1e9
    # parity of one more step against the oracle, on a sample of rows (rows are independent)
    last = args.warmup + args.steps
    step(last)
    torch.cuda.synchronize()
    sample = list(range(0, rows, max(1, rows // 8)))[:8]
    idx_s = routes[last % 8].cpu().numpy()[sample]
    w_last = w_host if last % rotation == 0 else O.fill_weights(sid, 778 + last % rotation - 1, k, n * E)
    ref = O.grouped_matmul_bt(np.ascontiguousarray(x_host[sample]), w_last, idx_s, len(sample), k, n, E, sid)
    got = y.cpu().numpy()[sample]
    xn = np.sqrt((x_host[sample].astype(np.float64) ** 2).sum(axis=1))
    wn = np.stack([O.row_norms(sid, w_last[int(e) * slab:(int(e) + 1) * slab], k, n) for e in idx_s])
    parity_max = float((np.abs(got - ref) / (xn[:, None] * wn)).max())
    if not parity_max <= 1e-3:
        raise SystemExit(f"MoE result differs from the oracle: {parity_max:.3e} of |x||w|")
    # end to end: activations and routing from pinned host memory, outputs back to the host
    x_pin = torch.from_numpy(x_host).pin_memory()
    r_pin = routes[1].cpu().pin_memory()
    y_pin = torch.empty((rows, n), dtype=torch.float32).pin_memory()
    x_st, r_st = torch.empty_like(x_dev), torch.empty_like(routes[0])

    def e2e_step(i):
        x_st.copy_(x_pin, non_blocking=True)
        r_st.copy_(r_pin, non_blocking=True)
        R.grouped_matmul(x_st, stacks[i % rotation], r_st, sid, n, E, out=y, workspace=wsb)
        y_pin.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    for i in range(3):
        e2e_step(i)
    e2e_n = max(2, min(args.steps, 50))
    t0 = time.perf_counter()
    for i in range(e2e_n):
        e2e_step(i)
    e2e_s = (time.perf_counter() - t0) / e2e_n
    peak, peak_src = measured_peaks()
    if prefill:
        pk = all_peaks()
        peak = pk["tf_burst"]
        peak_src = "measured (MEASURED_PEAKS.json bf16_tflops, burst)" if pk["measured"] else "fallback (1.59 PFLOP/s)"
    unit = "TFLOP/s" if prefill else "GB/s"
    e2e_value = step_flops / e2e_s / 1e12 if prefill else step_bytes / e2e_s / 1e9
    line = {
        "metric": "gemm_tflops" if prefill else "gemv_hbm_gbs", "value": value, "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": args.workload, "scheme": sch, "k": k, "n": n, "experts": E, "rows_per_step": rows,
                   "routing": ("rows dealt evenly over the experts, changing every step" if prefill
                               else "each row to a different expert, changing every step"),
                   "parity_max": parity_max,
                   "l2": f"rotating {rotation} expert stacks of {E * slab // 10**6} MB > 2 x 126 MB L2"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": rows * k * 4 + rows * 4,
                "d2h_bytes_per_step": rows * n * 4, "ms_per_step": e2e_s * 1e3,
                "api": "rlx_b200.grouped_matmul, pinned host buffers"},
        "gpu_launches": launches,
        "roofline": {"bound": "tensor" if prefill else "hbm", "achieved": value, "peak": peak, "unit": unit, "frac": value / peak,
                     "peak_source": peak_src,
                     "kernel": ("gemm_tcgen05_kernel in grouped mode (+ sort, tile table, gather, scatter)" if prefill
                                else "grouped matmul kernels of one step"),
                     "bytes_per_launch": step_bytes, "flops_per_launch": step_flops,
                     "avg_launch_us": ms_per_step * 1e3, "traffic": None},
    }
    if not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        srows = min(rows, 16)                                 # prefill: a sample of the rows, scaled (rows are independent)
        idx = routes[1].cpu().numpy()[:srows]
        xs = np.ascontiguousarray(x_host[:srows])
        O.grouped_matmul_bt(xs, w_host, idx, srows, k, n, E, sid)
        t0 = time.perf_counter(); reps = 0
        while time.perf_counter() - t0 < 6.0 and reps < 20:
            O.grouped_matmul_bt(xs, w_host, idx, srows, k, n, E, sid); reps += 1
        dt = (time.perf_counter() - t0) / reps * (rows / srows)
        line["cpu_baseline"] = {"value": (step_flops / dt / 1e12) if prefill else (step_bytes / dt / 1e9), "unit": unit,
                                "cores": cores, "kind": "port",
                                "sample": (f"{reps} passes over {srows} of the {rows} rows, scaled to a full step; " if prefill
                                           else f"{reps} full steps, ") +
                                          f"each expert's rows split over {cores} host threads "
                                          "(the reference runs them on one thread)"}
    print(json.dumps(line), flush=True)


def run_upload_workload(args, rank, world, local_rank):
    """GGUF file -> device: one step uploads every tensor of a synthetic 1 GB file of Q4_K blocks."""
    import struct
    import tempfile
    import numpy as np
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    import rlx_b200 as R
    from oracle import oracle as O      # input generation only
    torch.cuda.set_device(local_rank)
    k, n, count = 8192, 28672, 8                                  # eight 132 MB projections
    w = O.fill_weights(0, 9, k, n)
    tmp = tempfile.NamedTemporaryFile(suffix=".gguf", delete=False)
    names = [f"blk.{i}.ffn_up.weight" for i in range(count)]
    head = struct.pack("<IIQQ", 0x46554747, 3, count, 0)
    stride = (w.size + 31) // 32 * 32
    for i, nm in enumerate(names):
        b = nm.encode()
        head += struct.pack("<Q", len(b)) + b + struct.pack("<IQQIQ", 2, k, n, 12, i * stride)
    head += bytes((-len(head)) % 32)
    with open(tmp.name, "wb") as fh:
        fh.write(head)
        for _ in range(count):
            fh.write(w.tobytes() + bytes(stride - w.size))
    f = R.GgufFile(tmp.name)
    total = sum(f.get(nm).nbytes for nm in names)
    dst = [torch.empty(f.get(nm).nbytes, dtype=torch.uint8, device="cuda") for nm in names]
    from rlx_b200._lib import lib, check

    def step():
        for nm, d in zip(names, dst):
            check(lib.rlxq_gguf_upload_tensor(f._h, nm.encode(), d.data_ptr(), d.numel(), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()

    for _ in range(max(1, min(args.warmup, 3))):
        step()
    steps = max(2, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    ok = bool(np.array_equal(dst[-1].cpu().numpy(), w))
    # the reference's way: read the whole data segment into memory, slice, upload from pageable memory
    t0 = time.perf_counter()
    whole = np.fromfile(tmp.name, dtype=np.uint8, offset=f.data_start)
    for i, d in enumerate(dst):
        d.copy_(torch.from_numpy(whole[i * stride:i * stride + w.size]))
    torch.cuda.synchronize()
    ref_dt = time.perf_counter() - t0
    os.unlink(tmp.name)
    print(json.dumps({
        "metric": "gguf_upload_gbs", "value": total / dt / 1e9, "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8", "data": "synthetic",
        "config": {"workload": args.workload, "file": f"{count} Q4_K tensors of {k} x {n}, {total // 10**6} MB, page cache warm",
                   "path": "four reader threads: pread -> 8 MiB pinned buffers (two per reader) -> cudaMemcpyAsync on one stream"},
        "e2e": {"value": total / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": total, "d2h_bytes_per_step": 0,
                "matches_file": ok},
        "gpu_launches": 0,
        "cpu_baseline": {"value": total / ref_dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": "once: whole data segment read into memory, tensors sliced and copied from pageable memory "
                                   "(the reference's GgufFile::from_reader + set_param_bytes)"}}), flush=True)


def run_lm_workload(args, rank, world, local_rank):
    """Greedy token selection over a packed tied embedding: one rlxq_lm_head_argmax per step."""
    import torch
    if world != 1:
        raise SystemExit("the LM-head workload is single-GPU")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rlxq kernels have no CPU path")
    import rlx_b200 as R
    from oracle import oracle as O      # input generation and the cpu_baseline leg only
    sch, k, n = LM_WORKLOADS[args.workload]
    sid = SCHEME_IDS[sch]
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    wb = packed_bytes(sch, k, n)
    step_bytes = wb + k * 2 + 8
    rotation = max(2, -(-2 * L2_BYTES // wb) + 1)
    w_host = O.fill_weights(sid, 4242, k, n)
    wsets = [torch.from_numpy(w_host).to(dev)] + [torch.from_numpy(O.fill_weights(sid, 4243 + r, k, n)).to(dev)
                                                   for r in range(rotation - 1)]
    h_host = O.bf16_bits_to_f32(O.f32_to_bf16_bits(O.fill_normal(99, k))).ravel()
    h_dev = torch.from_numpy(h_host).to(dev).to(torch.bfloat16)
    ws = torch.empty(R.lm_head_workspace_bytes(sid, k, n, 1, 1), dtype=torch.uint8, device=dev)
    res = []

    def step(i, exact=True):
        res.append(R.gguf_tied_lm_argmax(h_dev, wsets[i % rotation], k, n, sid, exact=exact, workspace=ws))

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    launches0 = R.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            step(args.warmup + i)
    launches = R.launch_count() - launches0
    graph.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ev0.record(); graph.replay(); ev1.record()
    torch.cuda.synchronize()
    R.device_status()
    clocks = sampler.stop()
    ms_per_step = ev0.elapsed_time(ev1) / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    # the same without the exact re-ranking (logits carry the GEMV's rounding), for comparison
    gfast = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gfast):
        for i in range(args.steps):
            step(args.warmup + i, exact=False)
    gfast.replay()
    torch.cuda.synchronize()
    ev0.record(); gfast.replay(); ev1.record()
    torch.cuda.synchronize()
    fast_ms = ev0.elapsed_time(ev1) / args.steps
    # end to end: hidden state from pinned host memory, token id and logit back to the host
    h_pin = torch.from_numpy(h_host).to(torch.bfloat16).pin_memory()
    h_stage = torch.empty_like(h_dev)
    out_pin = torch.empty(2, dtype=torch.float32).pin_memory()     # token id (exact in f32 below 2^24) and logit

    def e2e_step(i):
        h_stage.copy_(h_pin, non_blocking=True)
        idx, val = R.gguf_tied_lm_argmax(h_stage, wsets[i % rotation], k, n, sid, exact=True, workspace=ws)
        out_pin[0:1].copy_(idx, non_blocking=True)
        out_pin[1:2].copy_(val, non_blocking=True)
        torch.cuda.synchronize()
        return int(out_pin[0]), float(out_pin[1])

    for i in range(3):
        e2e_step(i)
    t0 = time.perf_counter()
    e2e_n = max(2, min(args.steps, 50))
    for i in range(e2e_n):
        got = e2e_step(i)
    e2e_s = (time.perf_counter() - t0) / e2e_n
    first = e2e_step(0)
    peak, peak_src = measured_peaks()
    line = {
        "metric": "gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": args.workload, "scheme": sch, "n_embd": k, "n_vocab": n, "hidden": "bf16",
                   "selection": "argmax, winners re-evaluated in the reference's f32 order (RLXQ_LM_EXACT)",
                   "without_exact_reranking": {"ms_per_step": fast_ms, "value": step_bytes / (fast_ms * 1e-3) / 1e9},
                   "l2": f"rotating {rotation} distinct embedding copies ({rotation * wb // 10**6} MB) > 2 x 126 MB L2"},
        "clocks": clocks,
        "e2e": {"value": step_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": k * 2, "d2h_bytes_per_step": 16,
                "ms_per_step": e2e_s * 1e3, "api": "rlx_b200.gguf_tied_lm_argmax, pinned host buffers",
                "token": first[0], "logit": first[1]},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": "GB/s", "frac": value / peak,
                     "peak_source": peak_src, "kernel": "gemv_int_kernel (the logits); selection kernels included in the time",
                     "bytes_per_launch": step_bytes, "avg_launch_us": ms_per_step * 1e3, "traffic": None},
    }
    if not args.no_cpu_baseline:
        rows = 16384                                   # bounded sample: the first rows of the same embedding
        sub = w_host[:packed_bytes(sch, k, rows)]
        cores = os.cpu_count() or 1
        O.lm_argmax(h_host, sub, k, rows, sid)
        t0 = time.perf_counter(); reps = 0
        while time.perf_counter() - t0 < 6.0 and reps < 20:
            O.lm_argmax(h_host, sub, k, rows, sid); reps += 1
        dt = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": (packed_bytes(sch, k, rows) + k * 4) / dt / 1e9, "unit": "GB/s", "cores": cores,
                                "kind": "port", "sample": f"{reps} argmax passes over the first {rows} of {n} rows, rows split "
                                f"over {cores} host threads (the reference scans on one thread)"}
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + sorted(GEMM_WORKLOADS) + sorted(LM_WORKLOADS) + sorted(MOE_WORKLOADS) + [TP_WORKLOAD, "gguf_upload"],
                    help="default: the Q4_0 GEMV pair on one GPU, the tensor-parallel FFN on several")
    ap.add_argument("--impl", default="rlxq", choices=["rlxq", "reference"])
    ap.add_argument("--gemm-shape", default=None, help="m,k,n override for a GEMM workload (profiling a reduced case)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemv-kernel", type=int, default=0, choices=[0, 1, 2, 3, 4, 5],
                    help="force a GEMV kernel for the decode workloads (the library's gemv_kernel option): 0 automatic, "
                         "1 generic, 2 mma.sync tensor mode, 3 integer dp4a, 4 tcgen05, 5 integer MMA")
    ap.add_argument("--tp-fused", type=int, default=0, choices=[0, 1],
                    help="tensor-parallel workload: 1 the down projection pushes and sums inside its own kernel (the library's "
                         "tp_fused option), 0 a separate all-reduce launch follows it")
    ap.add_argument("--no-sweep", action="store_true",
                    help="default workload only: skip the `configs` list (the other configurations, one entry each)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload is None:
        args.workload = "q4_0_llama7b_ffn_gemv" if (world == 1 and args.gpus <= 1) else TP_WORKLOAD
    if args.workload in GEMM_WORKLOADS:
        run_gemm_workload(args, rank, world, local_rank)
        return
    if args.workload in LM_WORKLOADS:
        run_lm_workload(args, rank, world, local_rank)
        return
    if args.workload in MOE_WORKLOADS:
        run_moe_workload(args, rank, world, local_rank)
        return
    if args.workload == "gguf_upload":
        run_upload_workload(args, rank, world, local_rank)
        return
    if args.workload == TP_WORKLOAD:
        if args.impl == "reference":
            run_tp_reference_arm(args, rank, world)
        else:
            run_tp_workload(args, rank, world, local_rank)
        return

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rlxq kernels have no CPU path")
    import rlx_b200 as R
    from oracle import oracle as O      # input generation and the cpu_baseline leg only

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    sch, layers, act = WORKLOADS[args.workload]
    sid = SCHEME_IDS[sch]
    m = args.batch
    if args.gemv_kernel:
        R.set_option("gemv_kernel", args.gemv_kernel)
    kernel_name = {0: ("gemv_int_kernel, dp4a units (+ its activation quantiser)" if m == 1
                       else "gemv_int_kernel, integer-MMA units (+ its activation quantiser) where the shape allows, else gemv_staged_kernel"),
                   1: "gemv_generic_kernel", 2: "gemv_staged_kernel (+ its activation converter)",
                   3: "gemv_int_kernel, dp4a units (+ its activation quantiser)", 4: "gemv_tc_kernel",
                   5: "gemv_int_kernel, integer-MMA units (+ its activation quantiser)"}[args.gemv_kernel]
    act_t = torch.float32 if act == "f32" else torch.bfloat16
    act_bytes = 4 if act == "f32" else 2
    per_launch = algorithmic_bytes(sch, layers, m, act_bytes)
    step_bytes = sum(per_launch)
    w_step = sum(packed_bytes(sch, k, n) for k, n in layers)
    rotation = max(2, -(-2 * L2_BYTES // w_step) + 1)

    # ---- inputs resident in HBM: `rotation` independent weight sets, one activation per rank
    dev = torch.device("cuda", local_rank)
    wsets = []
    for r in range(rotation):
        wsets.append([torch.from_numpy(O.fill_weights(sid, 1000 + 100 * rank + 10 * r + i, k, n)).to(dev)
                      for i, (k, n) in enumerate(layers)])
    x_host = O.fill_normal(77 + rank, m * layers[0][0]).reshape(m, layers[0][0])
    x_dev = torch.from_numpy(x_host).to(dev).to(act_t)
    outs = [torch.empty((m, n), dtype=torch.float32, device=dev) for _, n in layers]
    ws_need = max(R.workspace_bytes(sid, m, k, n, 0 if act == "f32" or i else 1, 0) for i, (k, n) in enumerate(layers))
    ws = torch.empty(max(ws_need, 16), dtype=torch.uint8, device=dev)

    def step(i: int) -> None:
        cur = x_dev
        for li, (k, n) in enumerate(layers):
            R.matmul(cur, wsets[i % rotation][li], sid, n, out=outs[li], workspace=ws)
            cur = outs[li]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    sync_all()
    # The K timed steps are captured once into a CUDA graph (the reference's ExecMode::Graph does the
    # same with its step loop) so that the device, not the Python launch path, sets the pace.
    launches0 = R.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(args.steps):
            step(args.warmup + i)
    launches = R.launch_count() - launches0     # kernels per replay
    graph.replay()                              # one untimed replay on top of the W warm-up steps
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    ev0.record()
    graph.replay()
    ev1.record()
    sync_all()
    R.device_status()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        lt = torch.tensor([launches], dtype=torch.int64, device=dev)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt.item())
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the Graph / Session API with pinned host buffers
    g = R.Graph("bench")
    xi = g.input("x", [m, layers[0][0]], R.DType.F32 if act == "f32" else R.DType.BF16)
    cur, names = xi, []
    for li, (k, n) in enumerate(layers):
        p = g.param(f"w{li}", [packed_bytes(sch, k, n)])
        names.append(f"w{li}")
        cur = g.dequant_matmul_packed(cur, p, R.QuantScheme(sid), n)
    g.set_outputs([cur])
    compiled = []
    sess = R.Session(R.Device.Cuda, index=local_rank, exec_mode="graph")
    for r in range(rotation):
        c = sess.compile(g)
        for li, nm in enumerate(names):
            c.set_param_typed(nm, wsets[r][li].cpu().numpy(), R.DType.U8)
        compiled.append(c)
    x_pin = torch.from_numpy(x_host).to(act_t).pin_memory()
    y_pin = torch.empty((m, layers[-1][1]), dtype=torch.float32).pin_memory()
    h2d, d2h = x_pin.numel() * x_pin.element_size(), y_pin.numel() * 4
    dt_in = 0 if act == "f32" else 1

    bound = [c.bind_raw(["x"], [x_pin.data_ptr()], [h2d], [dt_in], y_pin.data_ptr(), d2h, 0) for c in compiled]

    def e2e_step(i: int) -> None:
        bound[i % rotation]()

    for i in range(args.warmup):
        e2e_step(i)
    sync_all()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(args.warmup + i)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = world * step_bytes / (e2e_s / args.steps) / 1e9
    # the e2e output must be the same numbers the resident path produced
    step(args.warmup + args.steps - 1)
    torch.cuda.synchronize()
    e2e_matches = bool(torch.equal(outs[-1].cpu(), y_pin))
    # the headline's own parity: both layers of the last weight set against the oracle, each on the input it had
    headline_parity = None
    if rank == 0:
        wl = wsets[(args.warmup + args.steps - 1) % rotation]
        headline_parity, cur_h = 0.0, x_host if act == "f32" else O.bf16_bits_to_f32(O.f32_to_bf16_bits(x_host)).reshape(m, -1)
        for li, (k, n) in enumerate(layers):
            wh = wl[li].cpu().numpy()
            ref = O.matmul_bt_mt(cur_h, wh, m, k, n, O.SCHEMES[sch])
            yh = outs[li].cpu().numpy()
            xn = np.sqrt((cur_h.astype(np.float64) ** 2).sum(axis=1))
            headline_parity = max(headline_parity, parity_ratio(yh, ref, xn, O.row_norms(O.SCHEMES[sch], wh, k, n)))
            cur_h = yh

    if rank == 0:
        peak, peak_src = measured_peaks()
        n_launch = len(layers) * args.steps
        avg_launch_s = ms * 1e-3 / n_launch
        bytes_per_launch = step_bytes / len(layers)
        achieved = bytes_per_launch / avg_launch_s / 1e9
        line = {
            "metric": "gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, sch, layers, act, rotation),
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s / args.steps * 1e3, "matches_resident_path": e2e_matches,
                    "api": "Session(Device.Cuda).compile(graph).run, pinned host buffers, ExecMode::Graph"},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "frac_of_nominal_8TBs": achieved / 8000.0,
                         "kernel": kernel_name, "bytes_per_launch": bytes_per_launch,
                         "avg_launch_us": avg_launch_s * 1e6,
                         "timing": "CUDA events over the timed region / launches (includes inter-launch gaps)",
                         "traffic": captured_traffic(args.workload, m)},
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(sch, layers, m, act)
        if world == 1 and not args.no_sweep and args.workload == "q4_0_llama7b_ffn_gemv" and m == 1 and not args.gemv_kernel:
            head = {"name": "cfg1 q4_0 llama7b ffn gemv pair m=1 (the headline)", "scheme": sch, "m": m,
                    "layers_k_to_n": [[k, n] for k, n in layers], "activations": act, "metric": "gemv_hbm_gbs",
                    "value": value, "unit": "GB/s", "ms": ms_per_step,
                    "roofline": {"bound": "hbm", "frac": achieved / peak, "peak": peak, "peak_kind": peak_src},
                    "parity_max": headline_parity, "parity_sample": "every output of both layers"}
            line["configs"] = sweep_all_configs(torch, R, O, dev, head)
        print(json.dumps(line), flush=True)
    if world > 1:
        finish_ranks(dist, torch)


if __name__ == "__main__":
    main()
